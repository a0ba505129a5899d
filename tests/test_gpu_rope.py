"""GPU parity of part 2 (RoPE on Q/K, int8 KV stores, paged copy, and the fused RoPE + int8 paged store)
against the CPU oracle and the golden vectors, through the operator shims over the C ABI.

Rotated bf16 outputs are compared bit-exactly where the oracle evaluates the same fp32 operation sequence
(products and sums rounded separately); int8 codes: +-1 LSB on <= 0.01 %."""
import pytest
import torch

from mcoplib_b200 import workloads as W
from oracle import compare as C
from oracle import ref_ops as R
from tests.golden_io import records
from tests.gpu_util import DEV, Canary, bits, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def op():
    from mcoplib_b200 import op as _op
    return _op


def _fused(op, d, ks, vs, is_neox=True):
    g = to_dev(d)
    kc = Canary(tuple(d["key_cache"].shape), torch.int8)
    vc = Canary(tuple(d["value_cache"].shape), torch.int8)
    v_before = g["value"].clone()
    op.rope_kv_store_int8(g["positions"], g["query"], g["key"], g["value"], d["head_size"], g["cos_sin_cache"], is_neox,
                          kc.t, vc.t, g["slot_mapping"], ks.to(DEV), vs.to(DEV))
    torch.cuda.synchronize()
    kc.check("key cache"); vc.check("value cache")
    assert torch.equal(g["value"], v_before)
    return g["query"].cpu(), g["key"].cpu(), kc.t.cpu(), vc.t.cpu()


def _oracle_fused(d, is_neox=True):
    Hkv, D = d["key_cache"].shape[2], d["head_size"]
    _, kr = R.rotary_embedding(d["positions"], d["query"], d["key"], D, d["cos_sin_cache"], is_neox)
    ks, vs = W.kv_scales(kr, d["value"], Hkv, D)
    q, k, kc, vc = R.rope_kv_store_int8(d["positions"], d["query"], d["key"], d["value"], D, d["cos_sin_cache"], is_neox,
                                        d["key_cache"], d["value_cache"], d["slot_mapping"], ks, vs)
    return ks, vs, q, k, kc, vc


def test_config2_fused_rope_kv_store(op):
    """Benchmark configuration 2 in full: 4096 tokens, 32/8 heads, D 128, fp32 cos/sin cache, 2048 blocks of 16."""
    d = W.rope_kv_inputs(4096, 32, 8, 128, 8192)
    ks, vs, q_ref, k_ref, kc_ref, vc_ref = _oracle_fused(d)
    q, k, kc, vc = _fused(op, d, ks, vs)
    C.assert_equal(bits(q), bits(q_ref), "query"); C.assert_equal(bits(k), bits(k_ref), "key")
    C.assert_codes(kc, kc_ref, "key cache"); C.assert_codes(vc, vc_ref, "value cache")
    # untouched slots stay zero; every written slot reaches the full code range for at least one head overall
    used = torch.zeros(2048 * 16, dtype=torch.bool); used[d["slot_mapping"]] = True
    assert int(kc.reshape(-1, 8 * 128)[~used].abs().max()) == 0
    assert int(kc.abs().max()) == 127 and int(vc.abs().max()) == 127


@pytest.mark.parametrize("tokens,hq,hkv,D", [(1, 1, 1, 64), (37, 4, 4, 128), (130, 8, 2, 96), (64, 16, 1, 256), (50, 6, 2, 32)])
@pytest.mark.parametrize("cache_dtype", [torch.float32, torch.bfloat16])
def test_fused_shapes_and_cache_dtypes(op, tokens, hq, hkv, D, cache_dtype):
    d = W.rope_kv_inputs(tokens, hq, hkv, D, 512, num_blocks=16)
    d["cos_sin_cache"] = d["cos_sin_cache"].to(cache_dtype)
    ks, vs, q_ref, k_ref, kc_ref, vc_ref = _oracle_fused(d)
    q, k, kc, vc = _fused(op, d, ks, vs)
    C.assert_equal(bits(q), bits(q_ref)); C.assert_equal(bits(k), bits(k_ref))
    C.assert_codes(kc, kc_ref); C.assert_codes(vc, vc_ref)


def test_fused_skips_negative_and_out_of_range_slots(op):
    d = W.rope_kv_inputs(64, 4, 2, 128, 512, num_blocks=8)
    d["slot_mapping"][::3] = -1
    ks, vs, q_ref, k_ref, kc_ref, vc_ref = _oracle_fused(d)
    q, k, kc, vc = _fused(op, d, ks, vs)
    C.assert_equal(bits(q), bits(q_ref)); C.assert_equal(bits(k), bits(k_ref))   # rotation still happens
    C.assert_equal(kc, kc_ref); C.assert_equal(vc, vc_ref)
    d2 = W.rope_kv_inputs(64, 4, 2, 128, 512, num_blocks=8)
    d2["slot_mapping"][5] = 8 * 16 + 3                                              # beyond the cache: skipped, not written
    keep = torch.ones(64, dtype=torch.bool); keep[5] = False
    ks, vs = W.kv_scales(R.rotary_embedding(d2["positions"], d2["query"], d2["key"], 128, d2["cos_sin_cache"], True)[1], d2["value"], 2, 128)
    from mcoplib_b200 import cabi
    assert cabi.load().mcop_device_error() == 0, "negative slots are the caller's no-store mark, not an error"
    _fused(op, d2, ks, vs)
    assert cabi.load().mcop_device_error() == cabi.DEVERR_SLOT, "a slot past the cache is skipped AND reported"


def test_fused_gptj_and_partial_rotation_use_the_generic_kernel(op):
    for is_neox, rot in [(False, 128), (True, 64), (False, 64)]:
        d = W.rope_kv_inputs(40, 4, 2, 128, 256, num_blocks=8)
        d["cos_sin_cache"] = W.cos_sin_cache(256, rot, 10000.0)
        ks, vs, q_ref, k_ref, kc_ref, vc_ref = _oracle_fused(d, is_neox)
        q, k, kc, vc = _fused(op, d, ks, vs, is_neox)
        C.assert_equal(bits(q), bits(q_ref)); C.assert_equal(bits(k), bits(k_ref))
        C.assert_codes(kc, kc_ref); C.assert_codes(vc, vc_ref)


@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("cache_dtype", [torch.bfloat16, torch.float32])
def test_vllm_rotary_embedding(op, is_neox, cache_dtype, golden):
    ns = getattr(torch.ops, op.torch_namespace)
    d = W.rope_kv_inputs(100, 8, 2, 128, 1024, num_blocks=8)
    cache = d["cos_sin_cache"].to(cache_dtype)
    q_ref, k_ref = R.rotary_embedding(d["positions"], d["query"], d["key"], 128, cache, is_neox)
    q, k = d["query"].to(DEV), d["key"].to(DEV)
    ns.rotary_embedding(d["positions"].to(DEV), q, k, 128, cache.to(DEV), is_neox)
    C.assert_equal(bits(q), bits(q_ref)); C.assert_equal(bits(k), bits(k_ref))
    # key=None, 3-D query view, 2-D positions
    q3 = d["query"].to(DEV).view(4, 25, 8, 128)
    ns.rotary_embedding(d["positions"].to(DEV).view(4, 25), q3, None, 128, cache.to(DEV), is_neox)
    C.assert_equal(bits(q3.reshape(100, -1)), bits(q_ref))
    # golden vectors produced by the reference's apply_rope_ref (fp32 form)
    if cache_dtype == torch.float32:
        for key, g in records(golden, "ref:benchmark/runners/mcoplib_mxbenchmark_batched_rotary_embedding_runners.py:apply_rope_ref"):
            if bool(g["is_neox"]) != is_neox:
                continue
            qq = g["query"].reshape(g["query"].shape[0], -1).to(DEV)
            ns.rotary_embedding(g["positions"].to(DEV), qq, None, 128, g["cos_sin_cache"].to(DEV), is_neox)
            C.assert_equal(bits(qq.reshape(g["out"].shape)), bits(g["out"]), key)


def test_packed_rotary_embedding(op, golden):
    (key, g), = records(golden, "ref:benchmark/runners/mcoplib_mxbenchmark_rotary_embeding_runners.py:_torch_rope_impl")
    n = g["packed_qkv"].shape[0]
    out = torch.full_like(g["packed_qkv"], 7.0).to(DEV)
    op.rotary_embedding(g["packed_qkv"].to(DEV), torch.tensor([n], dtype=torch.int32, device=DEV),
                        torch.tensor([0, n], dtype=torch.int32, device=DEV), torch.tensor([0], dtype=torch.int32, device=DEV),
                        g["cos"].to(DEV), g["sin"].to(DEV), out, g["q_head_num"], g["kv_head_num"])
    nqk = g["q_head_num"] + g["kv_head_num"]
    C.assert_equal(bits(out[:, :nqk]), bits(g["out"][:, :nqk]), key)
    assert bool((out[:, nqk:] == 7.0).all()), "V heads of the output must not be touched"
    # several sequences with cache offsets
    T, Hq, Hkv, D = 90, 6, 2, 128
    packed = W.per_token("randn", 30, 0, T, (Hq + 2 * Hkv) * D, torch.bfloat16).reshape(T, Hq + 2 * Hkv, D)
    accum = torch.tensor([0, 20, 21, 90], dtype=torch.int32); q_len = torch.tensor([20, 1, 69], dtype=torch.int32)
    cache_lens = torch.tensor([5, 400, 0], dtype=torch.int32)
    cs = W.cos_sin_cache(512, D, 500000.0)
    cos, sin = cs[:, :D // 2].contiguous(), cs[:, D // 2:].contiguous()
    base = torch.zeros_like(packed)
    ref = R.rotary_embedding_packed(packed, q_len, accum, cache_lens, cos, sin, base, Hq, Hkv)
    out = base.to(DEV)
    op.rotary_embedding(packed.to(DEV), q_len.to(DEV), accum.to(DEV), cache_lens.to(DEV), cos.to(DEV), sin.to(DEV), out, Hq, Hkv, 0)
    C.assert_equal(bits(out), bits(ref))


def test_fused_rope_fwd(op):
    S, H, D = 70, 8, 128
    qkv = W.per_token("randn", 31, 0, S, 3 * H * D, torch.bfloat16).reshape(S, 3, H, D)
    cs = W.cos_sin_cache(256, D, 10000.0)
    cos, sin = cs[:, :D // 2].bfloat16().contiguous(), cs[:, D // 2:].bfloat16().contiguous()
    idx = torch.randint(0, 256, (S,), generator=torch.Generator().manual_seed(1))
    for indexes in (None, idx):
        ref = R.fused_rope_fwd(qkv, cos, sin, indexes)
        g = qkv.to(DEV)
        ret = op.fused_rope_fwd(g, cos.to(DEV), sin.to(DEV), indexes.to(DEV) if indexes is not None else None, False)
        assert ret.data_ptr() == g.data_ptr()
        C.assert_equal(bits(g), bits(ref))
    with pytest.raises(RuntimeError):
        op.fused_rope_fwd(qkv.float().to(DEV), cos.to(DEV), sin.to(DEV), None, False)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_packed_and_plane_rope_through_the_pipelined_kernel(op, dtype):
    """From 2048 tokens on, mcoplib.op's packed rotary_embedding (positions derived from the sequence bounds, separate fp32 cos
    and sin tables, output to a second tensor) and fused_rope_fwd (Q and K planes of [S, 3, H, D], cos / sin tables of the
    element type) take the pipelined kernel: the two half rows of a position land side by side in the ring stage.
    Bit-exact against the oracle; V heads / the V plane untouched."""
    g = torch.Generator().manual_seed(33)
    D = 128
    cs = W.cos_sin_cache(8192, D, 500000.0)
    cos, sin = cs[:, :D // 2].contiguous(), cs[:, D // 2:].contiguous()
    if dtype == torch.bfloat16:   # the packed operator is bf16 only, as in the reference
        T, Hq, Hkv = 6000, 16, 4
        packed = torch.randn(T, Hq + 2 * Hkv, D, generator=g).to(dtype)
        accum = torch.tensor([0, 2500, 2501, 6000], dtype=torch.int32); q_len = torch.tensor([2500, 1, 3499], dtype=torch.int32)
        cache_lens = torch.tensor([5, 400, 0], dtype=torch.int32)
        base = torch.full_like(packed, 7.0)
        ref = R.rotary_embedding_packed(packed, q_len, accum, cache_lens, cos, sin, base, Hq, Hkv)
        out = base.to(DEV)
        op.rotary_embedding(packed.to(DEV), q_len.to(DEV), accum.to(DEV), cache_lens.to(DEV), cos.to(DEV), sin.to(DEV), out, Hq, Hkv, 0)
        assert _device_error() == 0
        C.assert_equal(bits(out), bits(ref))
    S, H = 4500, 8
    qkv = torch.randn(S, 3, H, D, generator=g).to(dtype)
    cos_t, sin_t = cos.to(dtype).contiguous(), sin.to(dtype).contiguous()
    idx = torch.randint(0, 8192, (S,), generator=g)
    for indexes in (None, idx):
        ref = R.fused_rope_fwd(qkv, cos_t, sin_t, indexes)
        gq = qkv.to(DEV)
        op.fused_rope_fwd(gq, cos_t.to(DEV), sin_t.to(DEV), indexes.to(DEV) if indexes is not None else None, False)
        assert _device_error() == 0
        C.assert_equal(bits(gq), bits(ref))


def test_fused_rope_fwd_force_bf16_attn(op):
    """force_bf16_attn on f16 data (op/fused_rope.cu:44-52): fp32 rotation of the f16 inputs, Q and K rounded once to bf16
    and stored in place, V keeps its f16 bits, the result is the same storage viewed as bf16."""
    S, H, D = 70, 8, 128
    qkv = W.per_token("randn", 32, 0, S, 3 * H * D, torch.float16).reshape(S, 3, H, D)
    cs = W.cos_sin_cache(256, D, 10000.0)
    cos, sin = cs[:, :D // 2].half().contiguous(), cs[:, D // 2:].half().contiguous()
    idx = torch.randint(0, 256, (S,), generator=torch.Generator().manual_seed(1))
    c, sn = cos[idx].float()[:, None, None, :], sin[idx].float()[:, None, None, :]
    x, y = qkv[:, :2, :, :D // 2].float(), qkv[:, :2, :, D // 2:].float()
    ref_x = (x * c - y * sn).bfloat16()     # products and difference rounded separately in fp32, one rounding to bf16
    ref_y = (y * c + x * sn).bfloat16()
    g = qkv.to(DEV)
    ret = op.fused_rope_fwd(g, cos.to(DEV), sin.to(DEV), idx.to(DEV), True)
    assert ret.dtype == torch.bfloat16 and ret.data_ptr() == g.data_ptr()
    C.assert_equal(bits(ret[:, :2, :, :D // 2]), bits(ref_x)); C.assert_equal(bits(ret[:, :2, :, D // 2:]), bits(ref_y))
    C.assert_equal(bits(g[:, 2]), bits(qkv[:, 2]))   # V: untouched f16 bits
    # with bf16 data the flag changes nothing
    qb = qkv.bfloat16()
    a = op.fused_rope_fwd(qb.to(DEV), cos.bfloat16().to(DEV), sin.bfloat16().to(DEV), idx.to(DEV), True)
    b = op.fused_rope_fwd(qb.to(DEV), cos.bfloat16().to(DEV), sin.bfloat16().to(DEV), idx.to(DEV), False)
    assert a.dtype == torch.bfloat16 and torch.equal(a, b)


def _fused_rope_bwd_literal(qkv, cos, sin, indexes):
    """kernel/fused_rope_kernel.h:172-176 written out: x' = x*c + y*s, y' = -x*s + y*c in fp32, one rounding."""
    S, _, H, D = qkv.shape
    idx = torch.arange(S) if indexes is None else indexes.long()
    c = cos[idx].float()[:, None, None, :]
    s = sin[idx].float()[:, None, None, :]
    out = qkv.clone()
    x, y = qkv[:, :2, :, :D // 2].float(), qkv[:, :2, :, D // 2:].float()
    out[:, :2, :, :D // 2] = (x * c + y * s).to(qkv.dtype)
    out[:, :2, :, D // 2:] = (-(x * s) + y * c).to(qkv.dtype)
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,H,D", [(70, 8, 128), (3000, 4, 64), (5, 3, 80)])
def test_fused_rope_bwd(op, dtype, S, H, D):
    qkv = W.per_token("randn", 37, 0, S, 3 * H * D, dtype).reshape(S, 3, H, D)
    cs = W.cos_sin_cache(4096, D, 10000.0)
    cos, sin = cs[:, :D // 2].to(dtype).contiguous(), cs[:, D // 2:].to(dtype).contiguous()
    idx = torch.randint(0, 4096, (S,), generator=torch.Generator().manual_seed(2))
    for indexes in (None, idx):
        ref = R.fused_rope_bwd(qkv, cos, sin, indexes)
        C.assert_equal(bits(ref), bits(_fused_rope_bwd_literal(qkv, cos, sin, indexes)))
        g = qkv.to(DEV)
        ret = op.fused_rope_bwd(g, cos.to(DEV), sin.to(DEV), indexes.to(DEV) if indexes is not None else None, False)
        assert ret.data_ptr() == g.data_ptr()
        C.assert_equal(bits(g), bits(ref))
        C.assert_equal(bits(g[:, 2]), bits(qkv[:, 2]))  # the V plane is not touched
        # the transposed rotation undoes the forward one up to the two roundings
        back = op.fused_rope_bwd(op.fused_rope_fwd(qkv.to(DEV), cos.to(DEV), sin.to(DEV), indexes.to(DEV) if indexes is not None else None, False),
                                 cos.to(DEV), sin.to(DEV), indexes.to(DEV) if indexes is not None else None, False)
        tol = 2.0 ** -6 if dtype == torch.bfloat16 else 2.0 ** -9
        assert torch.allclose(back.float().cpu(), qkv.float(), rtol=0, atol=tol * 8)
    with pytest.raises(RuntimeError):
        op.fused_rope_bwd(qkv.float().to(DEV), cos.to(DEV), sin.to(DEV), None, False)


def test_store_kv_cache_against_golden(op, golden):
    for key, g in records(golden, "ref:unit_test/test_store_kv.py:run_reference_impl"):
        kc = torch.zeros_like(g["k_cache"]).to(DEV); vc = torch.zeros_like(kc)
        op.store_kv_cache_cuda_interface(g["packed_qkv"].to(DEV), g["q_lens"].to(DEV), g["accum_q_lens"].to(DEV),
                                         g["cache_lens"].to(DEV), g["cache_slot_ids"].to(DEV), kc, vc, g["k_scale"].to(DEV),
                                         g["v_scale"].to(DEV), len(g["q_lens"]), g["q_head_num"], g["kv_head_num"])
        # reference tolerance atol=0.5 on integers == exact
        C.assert_equal(kc, g["k_cache"], key + " k"); C.assert_equal(vc, g["v_cache"], key + " v")
    # strided cache view
    g = records(golden, "ref:unit_test/test_store_kv.py:run_reference_impl")[1][1]
    big = torch.zeros(2, g["kv_head_num"], 48, 256, dtype=torch.int8, device=DEV)
    kc, vc = big[..., :128], big[..., 128:]
    op.store_kv_cache_cuda_interface(g["packed_qkv"].to(DEV), g["q_lens"].to(DEV), g["accum_q_lens"].to(DEV), g["cache_lens"].to(DEV),
                                     g["cache_slot_ids"].to(DEV), kc, vc, g["k_scale"].to(DEV), g["v_scale"].to(DEV), 2,
                                     g["q_head_num"], g["kv_head_num"])
    C.assert_equal(kc, g["k_cache"]); C.assert_equal(vc, g["v_cache"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 8, 128), (2, 1, 64), (3, 5, 80)])
def test_store_kv_cache_ragged_sequences(op, dtype, Hq, Hkv, D):
    """Sequences of 1 .. 37 tokens whose boundaries fall inside the groups of four consecutive tokens a thread of the
    vector kernel takes, tokens between two sequences that belong to none (q_len shorter than the gap to the next
    offset), non-zero cache lengths, a shuffled slot order; head_dim 80 takes the element kernel.  Bit-exact."""
    g = torch.Generator().manual_seed(5)
    q_lens = torch.tensor([1, 5, 37, 2, 16, 7, 3, 30], dtype=torch.int32)
    gaps = torch.tensor([0, 2, 0, 1, 0, 0, 3, 0], dtype=torch.int32)          # unowned tokens after each sequence
    accum = torch.zeros(len(q_lens) + 1, dtype=torch.int32)
    accum[1:] = torch.cumsum(q_lens + gaps, 0)
    T = int(accum[-1])
    cache_lens = torch.tensor([0, 3, 1, 0, 9, 2, 0, 4], dtype=torch.int32)
    slots = torch.randperm(len(q_lens), generator=g).to(torch.int32)
    max_len = 48
    qkv = (torch.randn(T, Hq + 2 * Hkv, D, generator=g) * 3).to(dtype)
    ks = 20 + 10 * torch.rand(Hkv, D, generator=g); vs = 20 + 10 * torch.rand(Hkv, D, generator=g)
    kc0 = torch.full((len(q_lens), Hkv, max_len, D), 55, dtype=torch.int8); vc0 = torch.full_like(kc0, -55)
    kc_ref, vc_ref = R.store_kv_cache(qkv, q_lens, accum[:-1], cache_lens, slots, kc0, vc0, ks, vs, Hq, Hkv)
    kc, vc = kc0.to(DEV), vc0.to(DEV)
    op.store_kv_cache_cuda_interface(qkv.to(DEV), q_lens.to(DEV), accum.to(DEV), cache_lens.to(DEV), slots.to(DEV), kc, vc,
                                     ks.to(DEV), vs.to(DEV), len(q_lens), Hq, Hkv)
    torch.cuda.synchronize()
    assert _device_error() == 0
    C.assert_equal(kc.cpu(), kc_ref, "k cache"); C.assert_equal(vc.cpu(), vc_ref, "v cache")


def test_reshape_and_cache_flash(op):
    ns = getattr(torch.ops, op.torch_namespace + "_cache_ops")
    T, Hkv, D, bs, nb = 200, 4, 128, 16, 32
    key = W.per_token("randn", 40, 0, T, Hkv * D, torch.bfloat16).reshape(T, Hkv, D)
    val = W.per_token("randn", 41, 0, T, Hkv * D, torch.bfloat16).reshape(T, Hkv, D)
    slots = torch.randperm(nb * bs, generator=torch.Generator().manual_seed(2))[:T].to(torch.int64)
    slots[7] = -1
    kc0 = torch.zeros(nb, bs, Hkv, D, dtype=torch.bfloat16)
    kc_ref, vc_ref = R.reshape_and_cache_flash(key, val, kc0, kc0.clone(), slots)
    one = torch.ones(1, device=DEV)
    for layout in ("NHD", "HND"):
        if layout == "NHD":
            kc = kc0.clone().to(DEV); vc = kc0.clone().to(DEV)
        else:  # [nb, Hkv, bs, D] storage viewed as [nb, bs, Hkv, D]
            kc = torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device=DEV).permute(0, 2, 1, 3)
            vc = torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device=DEV).permute(0, 2, 1, 3)
        ns.reshape_and_cache_flash(key.to(DEV), val.to(DEV), kc, vc, slots.to(DEV), "auto", one, one)
        C.assert_equal(bits(kc.contiguous()), bits(kc_ref), layout); C.assert_equal(bits(vc.contiguous()), bits(vc_ref), layout)
        # the reference's own check: gather back through the slot mapping
        ok = slots >= 0
        blk, off = (slots[ok] // bs).to(DEV), (slots[ok] % bs).to(DEV)
        assert torch.equal(kc[blk, off].cpu(), key[ok])
    with pytest.raises(RuntimeError):
        ns.reshape_and_cache_flash(key.to(DEV), val.to(DEV), kc, vc, slots.to(DEV), "fp8", one, one)


@pytest.mark.parametrize("T,Hkv,D,bs,dtype", [(5000, 8, 128, 16, torch.bfloat16), (2049, 2, 64, 8, torch.float16), (1500, 40, 128, 16, torch.bfloat16)])
def test_reshape_and_cache_flash_many_tokens(op, T, Hkv, D, bs, dtype):
    """From 1024 tokens on a thread of the flash-layout copy moves one 16-byte vector of K and of V for four tokens (40 heads
    of 128 are more vectors than a CTA has threads: the row-per-token kernel).  Scattered slots, negative slots, a slot
    past the cache (skipped, reported); bit-exact against the oracle, untouched cells keep their canary value."""
    ns = getattr(torch.ops, op.torch_namespace + "_cache_ops")
    g = torch.Generator().manual_seed(23)
    nb = (T + bs - 1) // bs + 5
    key = torch.randn(T, Hkv, D, generator=g).to(dtype); val = torch.randn(T, Hkv, D, generator=g).to(dtype)
    slots = torch.randperm(nb * bs, generator=g)[:T].to(torch.int64)
    slots[3] = -1; slots[T - 1] = -1
    ref_slots = slots.clone()
    slots[700] = nb * bs + 9; ref_slots[700] = -1
    kc0 = torch.full((nb, bs, Hkv, D), 7.0, dtype=dtype)
    kc_ref, vc_ref = R.reshape_and_cache_flash(key, val, kc0, kc0.clone(), ref_slots)
    kc, vc = kc0.to(DEV), kc0.clone().to(DEV)
    one = torch.ones(1, device=DEV)
    _device_error()
    ns.reshape_and_cache_flash(key.to(DEV), val.to(DEV), kc, vc, slots.to(DEV), "auto", one, one)
    from mcoplib_b200 import cabi
    assert _device_error() == cabi.DEVERR_SLOT
    C.assert_equal(bits(kc), bits(kc_ref), "key cache"); C.assert_equal(bits(vc), bits(vc_ref), "value cache")


def test_config4_rope_kv_full_size_properties(op):
    """Benchmark configuration 4's RoPE stage (32768 tokens, 64/8 heads, positions < 131072): properties over
    the whole output, the oracle on a sample of tokens."""
    T, Hq, Hkv, D = 32768, 64, 8, 128
    d = W.rope_kv_inputs(T, Hq, Hkv, D, 131072, gen_device=DEV)
    q0, k0 = d["query"].clone(), d["key"].clone()
    kr = k0.clone()
    op.vllm_rotary_embedding(d["positions"], q0.clone(), kr, D, d["cos_sin_cache"], True)
    ks, vs = W.kv_scales(kr, d["value"], Hkv, D)
    op.rope_kv_store_int8(d["positions"], d["query"], d["key"], d["value"], D, d["cos_sin_cache"], True, d["key_cache"],
                          d["value_cache"], d["slot_mapping"], ks, vs)
    assert torch.equal(d["key"], kr), "fused and unfused rotation agree bit for bit"
    # rotation preserves the norm of every (x, y) pair up to bf16 rounding
    def pair_norm(t, H):
        t = t.float().reshape(T, H, 2, D // 2)
        return (t[:, :, 0] ** 2 + t[:, :, 1] ** 2).sum(-1)
    assert torch.allclose(pair_norm(d["query"], Hq), pair_norm(q0, Hq), rtol=2e-2)
    # round trip: cache[slot] * scale reproduces the rotated K / the V to half a code
    blk, off = d["slot_mapping"] // 16, d["slot_mapping"] % 16
    kdq = d["key_cache"][blk, off].float() * ks.view(1, Hkv, 1)
    vdq = d["value_cache"][blk, off].float() * vs.view(1, Hkv, 1)
    assert float((kdq - d["key"].float().view(T, Hkv, D)).abs().div(ks.view(1, Hkv, 1)).max()) <= 0.5 + 1e-3
    assert float((vdq - d["value"].float().view(T, Hkv, D)).abs().div(vs.view(1, Hkv, 1)).max()) <= 0.5 + 1e-3
    assert int(d["key_cache"].abs().max()) == 127 and int(d["value_cache"].abs().max()) == 127
    # oracle on 128 sampled tokens
    idx = torch.arange(0, T, T // 128, device=DEV)
    q_ref, k_ref = R.rotary_embedding(d["positions"][idx].cpu(), q0[idx].cpu(), k0[idx].cpu(), D, d["cos_sin_cache"].cpu(), True)
    C.assert_equal(bits(d["query"][idx]), bits(q_ref)); C.assert_equal(bits(d["key"][idx]), bits(k_ref))


def test_c_abi_rope_called_directly(op):
    from mcoplib_b200 import cabi
    from tests.gpu_util import stream_ptr
    lib = cabi.load()
    d = W.rope_kv_inputs(64, 8, 2, 128, 512, num_blocks=8)
    ks, vs, q_ref, k_ref, kc_ref, vc_ref = _oracle_fused(d)
    g = to_dev(d); ksg, vsg = ks.to(DEV), vs.to(DEV)
    rc = lib.mcop_rope_kv_store_i8_paged(g["positions"].data_ptr(), g["query"].data_ptr(), g["key"].data_ptr(), g["value"].data_ptr(),
                                         g["cos_sin_cache"].data_ptr(), cabi.F32_CODE, 512, g["key_cache"].data_ptr(), g["value_cache"].data_ptr(),
                                         g["slot_mapping"].data_ptr(), ksg.data_ptr(), vsg.data_ptr(), 64, 8, 2, 128, 128, 8 * 128, 2 * 128,
                                         2 * 128, 16, 8, 1, cabi.BF16_CODE, stream_ptr())
    cabi.check(rc, lib)
    torch.cuda.synchronize()
    C.assert_equal(bits(g["query"]), bits(q_ref)); C.assert_codes(g["key_cache"], kc_ref); C.assert_codes(g["value_cache"], vc_ref)


def test_reshape_and_cache_split_layout(op):
    """torch.ops._C_cache_ops.reshape_and_cache: K as [blocks, heads, head_size/x, block_size, x], V as
    [blocks, heads, head_size, block_size] (op/vllm/cache_kernels.cu:133-190), negative slots skipped."""
    ns = getattr(torch.ops, op.torch_namespace + "_cache_ops")
    one = torch.ones(1, device=DEV)
    for dtype, x, T, Hkv, D, bs, nb in [(torch.bfloat16, 8, 200, 4, 128, 16, 32), (torch.float16, 4, 33, 2, 64, 8, 16),
                                       (torch.float32, 4, 50, 3, 32, 4, 64), (torch.bfloat16, 8, 40, 40, 128, 16, 8)]:
        key = W.per_token("randn", 42, 0, T, Hkv * D, dtype).reshape(T, Hkv, D)
        val = W.per_token("randn", 43, 0, T, Hkv * D, dtype).reshape(T, Hkv, D)
        slots = torch.randperm(nb * bs, generator=torch.Generator().manual_seed(3))[:T].to(torch.int64)
        slots[5] = -1
        kc0 = torch.full((nb, Hkv, D // x, bs, x), 7.0, dtype=dtype)
        vc0 = torch.full((nb, Hkv, D, bs), 7.0, dtype=dtype)
        kc_ref, vc_ref = R.reshape_and_cache(key, val, kc0, vc0, slots)
        kc, vc = kc0.to(DEV), vc0.to(DEV)
        # key/value as strided views of a wider tensor: the token stride is not heads * head_size
        wide = torch.zeros(T, 2 * Hkv * D + 16, dtype=dtype, device=DEV)
        wide[:, :Hkv * D] = key.reshape(T, -1).to(DEV)
        wide[:, Hkv * D:2 * Hkv * D] = val.reshape(T, -1).to(DEV)
        kview = wide[:, :Hkv * D].view(T, Hkv, D)
        vview = wide[:, Hkv * D:2 * Hkv * D].view(T, Hkv, D)
        ns.reshape_and_cache(kview, vview, kc, vc, slots.to(DEV), "auto", one, one)
        C.assert_equal(bits(kc), bits(kc_ref), f"key cache {dtype} x={x}")
        C.assert_equal(bits(vc), bits(vc_ref), f"value cache {dtype} x={x}")
        # gather back through the slot mapping, as the reference's runner checks the flash form
        ok = slots >= 0
        blk, off = (slots[ok] // bs), (slots[ok] % bs)
        back = kc.cpu()[blk, :, :, off, :].reshape(int(ok.sum()), Hkv, D)
        assert torch.equal(back, key[ok])
    with pytest.raises(RuntimeError):
        ns.reshape_and_cache(kview, vview, kc, vc, slots.to(DEV), "fp8", one, one)
    with pytest.raises(RuntimeError):   # a flash-layout cache is not a split-layout cache
        ns.reshape_and_cache(kview, vview, torch.zeros(8, 16, 40, 128, dtype=dtype, device=DEV), vc, slots.to(DEV), "auto", one, one)


@pytest.mark.parametrize("dtype,x,Hkv,D,bs", [(torch.bfloat16, 8, 8, 128, 16), (torch.float16, 8, 2, 64, 32), (torch.bfloat16, 4, 3, 128, 8),
                                              (torch.bfloat16, 8, 40, 128, 16)])
def test_reshape_and_cache_split_layout_runs_of_consecutive_slots(op, dtype, x, Hkv, D, bs):
    """The tiled kernel of the split layout writes a run of tokens with consecutive slots inside one block as aligned
    pieces of up to 16 bytes.  The slot map mixes what a scheduler produces: sequences whose slots run through several
    blocks starting at any offset of a block and at any token index, single tokens, a negative slot inside a run, a slot
    past the cache (skipped, reported), and a tail of scattered slots.  Bit-exact against the oracle; cells that no token
    maps to keep their canary value.  (40 heads of 128: a window does not fit shared memory, the row-per-token kernel.)"""
    ns = getattr(torch.ops, op.torch_namespace + "_cache_ops")
    one = torch.ones(1, device=DEV)
    nb = 64
    g = torch.Generator().manual_seed(17)
    runs = [(3, bs + 2), (2 * bs, bs), (5 * bs + bs - 1, 2), (9 * bs + 5, 1), (12 * bs, 3 * bs + 7), (20 * bs + 3, bs - 3), (30 * bs + 1, 29)]
    slots = torch.cat([torch.arange(s0, s0 + n) for s0, n in runs])
    used = set(slots.tolist())
    free = torch.tensor([s_ for s_ in range(nb * bs) if s_ not in used])
    tail = free[torch.randperm(free.numel(), generator=g)[:45]]
    slots = torch.cat([slots, tail]).to(torch.int64)
    slots[10] = -1                       # inside the first run
    slots[50] = nb * bs + 4              # past the cache: skipped and reported
    T = slots.numel()
    key = (torch.randn(T, Hkv, D, generator=g)).to(dtype); val = (torch.randn(T, Hkv, D, generator=g)).to(dtype)
    kc0 = torch.full((nb, Hkv, D // x, bs, x), 7.0, dtype=dtype); vc0 = torch.full((nb, Hkv, D, bs), 7.0, dtype=dtype)
    ref_slots = slots.clone(); ref_slots[50] = -1
    kc_ref, vc_ref = R.reshape_and_cache(key, val, kc0, vc0, ref_slots)
    kc, vc = kc0.to(DEV), vc0.to(DEV)
    _device_error()
    ns.reshape_and_cache(key.to(DEV), val.to(DEV), kc, vc, slots.to(DEV), "auto", one, one)
    from mcoplib_b200 import cabi
    assert _device_error() == cabi.DEVERR_SLOT
    C.assert_equal(bits(kc), bits(kc_ref), "key cache"); C.assert_equal(bits(vc), bits(vc_ref), "value cache")


def _device_error():
    from mcoplib_b200 import cabi
    torch.cuda.synchronize()
    return cabi.load().mcop_device_error()


@pytest.mark.parametrize("T", [48, 4096])   # token-per-CTA kernel, pipelined kernel
def test_out_of_range_position_skips_the_token_and_is_reported(op, T):
    """A position outside the cos/sin table never becomes an address: the token (and nothing else) is left untouched,
    nothing is stored for it, and the device error word carries MCOP_DEVERR_POSITION."""
    from mcoplib_b200 import cabi
    d = W.rope_kv_inputs(T, 8, 2, 128, 512, num_blocks=max(8, T // 16))
    ks, vs, q_ref, k_ref, kc_ref, vc_ref = _oracle_fused(d)
    assert _device_error() == 0
    bad = [3, T - 2]
    pos = d["positions"].clone()
    pos[bad[0]] = 512          # one past the table
    pos[bad[1]] = -1
    g = to_dev(d)
    q0, k0 = g["query"].clone(), g["key"].clone()
    kc = Canary(tuple(d["key_cache"].shape), torch.int8); vc = Canary(tuple(d["value_cache"].shape), torch.int8)
    op.rope_kv_store_int8(pos.to(DEV), g["query"], g["key"], g["value"], 128, g["cos_sin_cache"], True, kc.t, vc.t,
                          g["slot_mapping"], ks.to(DEV), vs.to(DEV))
    assert _device_error() == cabi.DEVERR_POSITION
    assert _device_error() == 0, "reading the word clears it"
    kc.check("key cache"); vc.check("value cache")
    good = torch.ones(T, dtype=torch.bool); good[bad] = False
    C.assert_equal(bits(g["query"].cpu()[good]), bits(q_ref[good]), "other tokens rotate as usual")
    C.assert_equal(bits(g["key"].cpu()[good]), bits(k_ref[good]))
    assert torch.equal(g["query"][bad], q0[bad]) and torch.equal(g["key"][bad], k0[bad]), "the bad tokens are untouched"
    # cache: the bad tokens' slots keep their zeros, every other slot holds the oracle's codes
    slots = d["slot_mapping"]
    kcc, vcc = kc.t.cpu().view(-1, 2, 128), vc.t.cpu().view(-1, 2, 128)
    assert int(kcc[slots[bad]].abs().max()) == 0 and int(vcc[slots[bad]].abs().max()) == 0
    C.assert_codes(kcc[slots[good]], kc_ref.view(-1, 2, 128)[slots[good]]); C.assert_codes(vcc[slots[good]], vc_ref.view(-1, 2, 128)[slots[good]])
    # the unfused operator checks the same way
    q2 = q0.clone()
    op.vllm_rotary_embedding(pos.to(DEV), q2, None, 128, g["cos_sin_cache"], True)
    assert _device_error() == cabi.DEVERR_POSITION
    assert torch.equal(q2[bad], q0[bad])
    # and a following normal call is exact
    g2 = to_dev(d)
    op.vllm_rotary_embedding(g2["positions"], g2["query"], g2["key"], 128, g2["cos_sin_cache"], True)
    assert _device_error() == 0
    C.assert_equal(bits(g2["query"]), bits(q_ref))


def test_out_of_range_slot_is_skipped_and_reported(op):
    from mcoplib_b200 import cabi
    d = W.rope_kv_inputs(64, 8, 2, 128, 512, num_blocks=8)
    ks, vs, q_ref, k_ref, kc_ref, vc_ref = _oracle_fused(d)
    slots = d["slot_mapping"].clone()
    slots[10] = 8 * 16          # one past the cache
    g = to_dev(d)
    kc = Canary(tuple(d["key_cache"].shape), torch.int8); vc = Canary(tuple(d["value_cache"].shape), torch.int8)
    op.rope_kv_store_int8(g["positions"], g["query"], g["key"], g["value"], 128, g["cos_sin_cache"], True, kc.t, vc.t,
                          slots.to(DEV), ks.to(DEV), vs.to(DEV))
    assert _device_error() == cabi.DEVERR_SLOT
    kc.check("key cache"); vc.check("value cache")
    C.assert_equal(bits(g["query"]), bits(q_ref), "rotation does not depend on the slot")
    assert int(kc.t.cpu().view(-1, 2, 128)[d["slot_mapping"][10]].abs().max()) == 0
    # paged copy
    ns = getattr(torch.ops, op.torch_namespace + "_cache_ops")
    key = g["key"].view(64, 2, 128); one = torch.ones(1, device=DEV)
    kcf = Canary((8, 16, 2, 128), torch.bfloat16); vcf = Canary((8, 16, 2, 128), torch.bfloat16)
    ns.reshape_and_cache_flash(key, key, kcf.t, vcf.t, slots.to(DEV), "auto", one, one)
    assert _device_error() == cabi.DEVERR_SLOT
    kcf.check("flash cache"); vcf.check("flash cache")


def test_store_kv_bad_slot_or_length_is_skipped_and_reported(op, golden):
    from mcoplib_b200 import cabi
    key, g = records(golden, "ref:unit_test/test_store_kv.py:run_reference_impl")[0]
    kc = Canary(tuple(g["k_cache"].shape), torch.int8); vc = Canary(tuple(g["v_cache"].shape), torch.int8)
    args = lambda slots, lens: (g["packed_qkv"].to(DEV), g["q_lens"].to(DEV), g["accum_q_lens"].to(DEV), lens.to(DEV), slots.to(DEV),
                                kc.t, vc.t, g["k_scale"].to(DEV), g["v_scale"].to(DEV), len(g["q_lens"]), g["q_head_num"], g["kv_head_num"])
    bad_slots = g["cache_slot_ids"].clone(); bad_slots[0] = g["k_cache"].shape[0]
    op.store_kv_cache_cuda_interface(*args(bad_slots, g["cache_lens"]))
    assert _device_error() == cabi.DEVERR_KV_INDEX
    kc.check("k cache"); vc.check("v cache")
    bad_lens = g["cache_lens"].clone(); bad_lens[0] = g["k_cache"].shape[2]
    op.store_kv_cache_cuda_interface(*args(g["cache_slot_ids"], bad_lens))
    assert _device_error() == cabi.DEVERR_KV_INDEX
    kc.check("k cache"); vc.check("v cache")
    kc.t.zero_(); vc.t.zero_()
    op.store_kv_cache_cuda_interface(*args(g["cache_slot_ids"], g["cache_lens"]))
    assert _device_error() == 0
    C.assert_equal(kc.t, g["k_cache"], key + " k"); C.assert_equal(vc.t, g["v_cache"], key + " v")


def test_bounded_wait_runs_out_and_is_reported(op):
    """The bounded-wait path of the pipeline kernels, exercised without any copy in flight: the self-test kernel arms a
    stage that nothing fills, its wait runs out after a few thousand tries, the code is recorded, the drain runs, the
    kernel returns; the context stays usable and the next operator call is exact."""
    from mcoplib_b200 import cabi
    from tests.gpu_util import stream_ptr
    lib = cabi.load()
    assert _device_error() == 0
    cabi.check(lib.mcop_selftest_wait_timeout(2048, stream_ptr()), lib)
    assert _device_error() == cabi.DEVERR_SELFTEST
    assert _device_error() == 0
    d = W.rope_kv_inputs(4096, 8, 2, 128, 512, num_blocks=256)   # a pipelined kernel right after
    ks, vs, q_ref, k_ref, kc_ref, vc_ref = _oracle_fused(d)
    q, k, kc, vc = _fused(op, d, ks, vs)
    C.assert_equal(bits(q), bits(q_ref)); C.assert_codes(kc, kc_ref)
    assert _device_error() == 0
