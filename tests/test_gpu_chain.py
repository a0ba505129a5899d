"""The chained configuration-5 path (norm + quant -> softmax top-2 of 8 -> scatter + quant -> weighted gather, every stage fed
by the stage before) at the size ONE rank of an 8-GPU run handles, 32,768 tokens x 7168, against the CPU oracle: router ids
and the scatter permutation on all tokens / rows, codes, scales, scatter rows and gathered rows on a sample of 1024 tokens.
This is the check `bench.py --verify` runs on every rank; here it runs on one GPU for the first and the last shard of the
8-GPU split (the token offset changes the generated rows, not the kernels)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rank", [0, 7])
def test_chain5_shard_of_an_8_gpu_run_matches_the_oracle(rank):
    import bench
    from mcoplib_b200 import cabi, op
    tokens = 262144 // 8
    v = bench.verify_chain5(op, tokens, rank * tokens, torch.device("cuda", 0), 7168)
    assert v["mismatches"] == 0, v["detail"]
    assert v["sampled_tokens"] == 1024 and v["tokens"] == tokens and v["rows"] == 2 * tokens
    torch.cuda.synchronize()
    assert cabi.load().mcop_device_error() == 0


def test_digest_is_additive_over_shards():
    import bench
    g = torch.Generator().manual_seed(0)
    v = torch.randint(-128, 128, (1000, 64), generator=g).to(torch.int8).cuda()
    whole = bench._digest(v, 0)
    parts = sum(bench._digest(v[a:b], a) for a, b in ((0, 300), (300, 301), (301, 1000))) % bench.DIGEST_MOD
    assert whole == parts
    v[5, 3] += 1
    assert bench._digest(v, 0) != whole
