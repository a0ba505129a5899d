"""Host-side logic of the multi-GPU path on CPU: shard ranges, the shard-invariant input generator, and a
world_size-2 gloo run in which every rank processes its own token range (with the CPU oracle standing in for the
kernels) and the gathered result equals the single-process result bit for bit."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mcoplib_b200 import workloads as W
from mcoplib_b200.sharding import gather_for_verification, max_over_ranks, shard_range
from oracle import ref_ops as R


def test_shard_range_partitions_the_tokens():
    for tokens in (0, 1, 7, 4096, 262144, 262145):
        for world in (1, 2, 3, 8):
            spans = [shard_range(tokens, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == tokens
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)


def test_generator_is_shard_invariant():
    full = W.per_token("randn", 3, 0, 10000, 96, torch.bfloat16)
    for t0, t1 in [(0, 4096), (4000, 4200), (4096, 10000), (9999, 10000)]:
        assert torch.equal(W.per_token("randn", 3, t0, t1, 96, torch.bfloat16), full[t0:t1])
    pos = W.per_token("randint", 5, 0, 9000, 0, torch.int64, high=8192)
    assert torch.equal(W.per_token("randint", 5, 5000, 9000, 0, torch.int64, high=8192), pos[5000:])
    assert int(pos.max()) < 8192 and int(pos.min()) >= 0
    # different tensors / seeds / chunks are different streams
    assert not torch.equal(W.per_token("randn", 4, 0, 64, 96, torch.bfloat16), full[:64])
    assert not torch.equal(W.per_token("randn", 3, 0, 64, 96, torch.bfloat16, seed=1), full[:64])


def test_algorithmic_byte_counts():
    assert W.norm_quant_bytes(256, 4096) == 7_349_248
    b = W.chain5_bytes(262144)
    assert b["norm_quant"] == 13_154_400_256 and b["softmax_topk"] == 12_582_912
    assert b["scatter"] == 7_524_810_752 and b["gather"] == 11_276_386_304
    assert W.gate_bytes(8192, 256, 8) == 8_913_920
    assert W.scatter_bytes(8192, 7168, 256, 8) == 595_591_168
    assert W.gather_bytes(8192, 7168, 8, False) == 1_057_226_752 and W.gather_bytes(8192, 7168, 8, True) == 1_174_667_264


def _chain(x, res, w, logits, smooth, y, E, k):
    q, s, r = R.rms_norm_dynamic_per_token_quant(x, w, 1e-6, residual=res)
    tw, ids = R.moe_softmax_topk(logits, k)
    rows, rs, r2t, cnt, st, t2r = R.moe_scatter_dynamic_quant(x, ids, tw, smooth, E)
    out = R.moe_gather_weighted(y, r2t, ids, tw, st, torch.zeros(x.shape, dtype=torch.bfloat16), False)
    return q, s, r, ids, out, cnt


def _worker(rank, world, port, tokens, H, E, k, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    t0, t1 = shard_range(tokens, rank, world)
    n = t1 - t0
    d = W.norm_quant_inputs(n, H, t0=t0)
    logits = W.router_inputs(n, E, t0=t0)["logits"]
    dd = W.dispatch_inputs(n, H, E, k, t0=t0, with_hidden=False)
    q, s, r, ids, out, cnt = _chain(d["x"], d["residual"], d["weight"], logits, dd["smooth"], dd["y"], E, k)
    full = {name: gather_for_verification(t, tokens) for name, t in dict(q=q, s=s, r=r, ids=ids, out=out).items()}
    total_cnt = cnt.clone()
    dist.all_reduce(total_cnt)
    slowest = max_over_ranks(float(rank + 1), torch.device("cpu"))
    if rank == 0:
        full["cnt"] = total_cnt
        full["slowest"] = torch.tensor(slowest)
        torch.save(full, result_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_gloo_run_equals_single_process(tmp_path):
    tokens, H, E, k = 777, 256, 8, 2     # odd token count: the ranks hold 389 and 388 tokens
    path = str(tmp_path / "gathered.pt")
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, tokens, H, E, k, path), nprocs=2, join=True)
    got = torch.load(path)
    d = W.norm_quant_inputs(tokens, H)
    logits = W.router_inputs(tokens, E)["logits"]
    dd = W.dispatch_inputs(tokens, H, E, k, with_hidden=False)
    q, s, r, ids, out, cnt = _chain(d["x"], d["residual"], d["weight"], logits, dd["smooth"], dd["y"], E, k)
    assert torch.equal(got["q"], q) and torch.equal(got["s"], s) and torch.equal(got["ids"], ids)
    assert torch.equal(got["r"].view(torch.int16), r.view(torch.int16))
    # the weighted gather consumes y rows in the rank-local (expert, token) order, so y differs per sharding;
    # what must agree is everything that is a per-token function of the inputs:
    assert torch.equal(got["cnt"], cnt)
    assert float(got["slowest"]) == 2.0
