"""moe_sum and moe_align_block_size (the token-major combine and the block-aligned index preparation of the
block-sparse expert GEMM; op/vllm/moe/moe_align_sum_kernels.cu).

CPU part: the oracle restatements are pinned to the constructions the reference's own benchmark runners check
against (benchmark/runners/mcoplib_mxbenchmark_moe_align_block_size_runners.py:62-107: bincount, padded ranges,
every expert's range sorted before comparing; mcoplib_mxbenchmark_moe_sum_runners.py:33-40: input.sum(dim=1)).
GPU part: the CUDA path through the shims over the C ABI against the oracle - indices bit-exact, sums bit-exact for
top-k 2..4 (running sum in the element type) and for the fp32-accumulated form."""
import pytest
import torch

from oracle import compare as C
from oracle import ref_ops as R

DEV = "cuda:0"


def _runner_reference(topk_ids, num_experts, block_size, max_padded):
    """The expected tensors as the reference's runner builds them (written out from its description: bincount per
    expert, counts rounded up to the block size, ranges laid out back to back)."""
    flat = topk_ids.flatten().long()
    n = flat.numel()
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + block_size - 1) // block_size * block_size
    sorted_ids = torch.full((max_padded,), n, dtype=torch.int32)
    expert_ids = torch.full((max_padded // block_size,), -1, dtype=torch.int32)
    off = 0
    for e in range(num_experts):
        idx = (flat == e).nonzero(as_tuple=True)[0]
        sorted_ids[off:off + idx.numel()] = idx.to(torch.int32)
        expert_ids[off // block_size:(off + int(padded[e])) // block_size] = e
        off += int(padded[e])
    return sorted_ids, expert_ids, torch.tensor([off], dtype=torch.int32)


@pytest.mark.parametrize("T,k,E,bs", [(2048, 2, 8, 64), (77, 8, 256, 16), (1, 4, 64, 128), (300, 6, 60, 32)])
def test_oracle_align_matches_runner_construction(T, k, E, bs):
    g = torch.Generator().manual_seed(T + E)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)  # experts may repeat inside a token, as in the runner
    cap = T * k + E * bs
    s, e, tot = R.moe_align_block_size(ids, E, bs, cap)
    rs, re, rtot = _runner_reference(ids, E, bs, cap)
    C.assert_equal(s, rs)
    C.assert_equal(tot, rtot)
    used = int(tot) // bs
    C.assert_equal(e[:used], re[:used])
    assert (e[used:] == 0).all()  # the kernel's fill of the unused blocks (the runner pre-fills -1 there)


def test_oracle_align_expert_map_and_invalid_ids():
    ids = torch.tensor([[0, 5], [7, 2], [9, -1], [2, 2]], dtype=torch.int32)
    emap = torch.tensor([1, -1, 0, -1, -1, 3, -1, -1], dtype=torch.int32)
    s, e, tot = R.moe_align_block_size(ids, 8, 2, 8 + 16, emap)
    # local expert 0 <- global 2 (entries 3, 6, 7), local 1 <- global 0 (entry 0), local 3 <- global 5 (entry 1)
    assert s[:10].tolist() == [3, 6, 7, 8, 0, 8, 1, 8, 8, 8]
    assert e[:4].tolist() == [0, 0, 1, 3] and int(tot) == 8


@pytest.mark.parametrize("k", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_oracle_moe_sum_against_framework_sum(k, dtype):
    x = torch.randn(16, k, 128, generator=torch.Generator().manual_seed(k)).to(dtype)
    ref = R.moe_sum(x)
    lib = x.sum(dim=1)
    # the framework accumulates in fp32 and rounds once; the per-add rounding of top-k 3 and 4 may differ by an ulp
    tol = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -20}[dtype]
    assert torch.allclose(ref.float(), lib.float(), rtol=tol, atol=8 * tol)  # an ulp of a partial sum of magnitude <= 8
    if k <= 2:
        C.assert_equal(ref.float(), lib.float())


# ---------------------------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def op():
    from mcoplib_b200 import op as _op
    return _op


def _align_gpu(op, ids, E, bs, cap, emap=None, via_torch_ops=False):
    s = torch.full((cap,), -7, dtype=torch.int32, device=DEV)
    e = torch.full(((cap + bs - 1) // bs if bs > 0 else 1,), -7, dtype=torch.int32, device=DEV)
    tot = torch.full((1,), -7, dtype=torch.int32, device=DEV)
    fn = op.moe_align_block_size
    if via_torch_ops:
        fn = getattr(torch.ops, op.torch_moe_namespace).moe_align_block_size
    fn(ids.to(DEV), E, bs, s, e, tot, emap.to(DEV) if emap is not None else None)
    return s.cpu(), e.cpu(), tot.cpu()


@gpu
@pytest.mark.parametrize("T,k,E,bs", [(2048, 2, 8, 64), (77, 8, 256, 16), (1, 4, 64, 128), (300, 6, 60, 32),
                                      (8192, 8, 256, 64), (70000, 2, 8, 128), (513, 1, 1000, 8), (5, 2, 128, 64)])
def test_align_block_size_gpu(op, T, k, E, bs):
    g = torch.Generator().manual_seed(T * 7 + E)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    cap = T * k + E * bs
    ref = R.moe_align_block_size(ids, E, bs, cap)
    for via in (False, True):
        out = _align_gpu(op, ids, E, bs, cap, via_torch_ops=via)
        for a, b in zip(out, ref):
            C.assert_equal(a, b)


@gpu
def test_align_block_size_gpu_map_invalid_and_dtypes(op):
    E, bs, T, k = 64, 16, 1000, 4
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(-2, E + 3, (T, k), generator=g, dtype=torch.int32)  # some ids out of range
    emap = torch.randint(-1, E, (E,), generator=g, dtype=torch.int32)        # some experts not on this rank, some shared
    cap = T * k + E * bs
    ref = R.moe_align_block_size(ids, E, bs, cap, emap)
    for dt in (torch.int32, torch.int64, torch.int16):
        out = _align_gpu(op, ids.to(dt), E, bs, cap, emap)
        for a, b in zip(out, ref):
            C.assert_equal(a, b)
    # a sorted buffer that is too short is never overrun (a guard word behind it keeps its value)
    short = cap // 2
    buf = torch.full((short + 64,), -7, dtype=torch.int32, device=DEV)
    e = torch.zeros(((short + bs - 1) // bs,), dtype=torch.int32, device=DEV)
    tot = torch.zeros(1, dtype=torch.int32, device=DEV)
    op.moe_align_block_size(ids.to(DEV), E, bs, buf[:short], e, tot, emap.to(DEV))
    assert (buf[short:] == -7).all()
    C.assert_equal(buf[:short].cpu(), ref[0][:short])
    # empty routing
    out = _align_gpu(op, torch.zeros(0, k, dtype=torch.int32), E, bs, E * bs)
    assert (out[0] == 0).all() and (out[1] == 0).all() and int(out[2]) == 0
    with pytest.raises(RuntimeError):
        _align_gpu(op, ids, E, 0, cap)
    with pytest.raises(RuntimeError):
        _align_gpu(op, ids, 1024, bs, cap)


@gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T,k,H", [(16, 2, 128), (333, 3, 7168), (64, 4, 4096), (50, 8, 2048), (7, 1, 512), (9, 6, 100), (12, 2, 36)])
def test_moe_sum_gpu(op, dtype, T, k, H):
    x = torch.randn(T, k, H, generator=torch.Generator().manual_seed(T + k)).to(dtype)
    ref = R.moe_sum(x)
    out = torch.full((T, H), float("nan"), dtype=dtype, device=DEV)
    op.moe_sum(x.to(DEV), out)
    C.assert_equal(out.cpu().view(torch.int16 if dtype != torch.float32 else torch.int32),
                   ref.view(torch.int16 if dtype != torch.float32 else torch.int32))
    out2 = torch.empty_like(out)
    getattr(torch.ops, op.torch_moe_namespace).moe_sum(x.to(DEV), out2)
    assert torch.equal(out, out2)
    # the check of the reference's runner: the framework's own sum over dim 1, to rounding
    tol = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -20}[dtype]
    assert torch.allclose(out.float().cpu(), x.sum(dim=1).float(), rtol=tol, atol=8 * tol)  # an ulp of a partial sum of magnitude <= 8


def test_oracle_moe_sum_reduce_against_the_reference_test_formula():
    # unit_test/test_moe_sum_reduce_triton.py: torch.sum(input, dim=1) * factor, DeepSeek shape 32 x 6 x 2048 fp16, cosine similarity
    x = torch.randn(32, 6, 2048, generator=torch.Generator().manual_seed(0)).half()
    for factor in (1.0, 2.5):
        ref = R.moe_sum_reduce(x, factor)
        lib = torch.sum(x, dim=1) * factor
        cos = torch.nn.functional.cosine_similarity(ref.flatten().float(), lib.flatten().float(), dim=0)
        assert cos > 0.99999
        assert torch.allclose(ref.float(), lib.float(), rtol=2.0 ** -9, atol=2.0 ** -9)


@gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T,k,H,factor", [(32, 6, 2048, 1.0), (300, 8, 7168, 2.5), (257, 2, 4096, 0.3), (5, 1, 520, 2.5), (9, 3, 100, 1.7)])
def test_moe_sum_reduce_gpu(op, dtype, T, k, H, factor):
    x = torch.randn(T, k, H, generator=torch.Generator().manual_seed(T + k)).to(dtype)
    ref = R.moe_sum_reduce(x, factor)
    out = torch.full((T, H), float("nan"), dtype=dtype, device=DEV)
    op.moe_sum_reduce(x.to(DEV), out, factor)
    view = torch.int16 if dtype != torch.float32 else torch.int32
    C.assert_equal(out.cpu().view(view), ref.view(view))
    with pytest.raises(RuntimeError):
        op.moe_sum_reduce(x.to(DEV), out[:, :H - 4], factor)


@gpu
def test_moe_sum_rejects(op):
    x = torch.zeros(4, 2, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError):
        op.moe_sum(x, torch.zeros(4, 64, dtype=torch.float16, device=DEV))
    with pytest.raises(RuntimeError):
        op.moe_sum(x[:, :, :32], torch.zeros(4, 32, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(RuntimeError):
        op.moe_sum(x.cpu(), torch.zeros(4, 64, dtype=torch.bfloat16))
