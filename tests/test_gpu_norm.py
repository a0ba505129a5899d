"""GPU parity of part 1 (residual add + RMSNorm + per-token int8 quant) against the CPU oracle and the
golden vectors.  Every call goes through the operator shims, i.e. through the C ABI of libmcop_b200.so.

Tolerances (oracle/compare.py): int8 codes +-1 LSB on <= 0.01 % of elements; scales and bf16 outputs
1e-2 relative / 1e-3 absolute; the in-place residual is bit-exact."""
import pytest
import torch

from mcoplib_b200 import workloads as W
from oracle import compare as C
from oracle import ref_ops as R
from tests.golden_io import records
from tests.gpu_util import DEV, Canary, bits

pytestmark = pytest.mark.gpu

FLT_EPSILON = 1.1920928955078125e-07


def _device_error_word():
    from mcoplib_b200 import cabi
    torch.cuda.synchronize()
    return cabi.load().mcop_device_error()


@pytest.fixture(scope="module")
def op():
    from mcoplib_b200 import op as _op
    return _op


def _run_a2(op, x, w, res, scale_ub=None):
    T, H = x.shape
    out = Canary((T, H), torch.int8)
    sc = Canary((T, 1), torch.float32)
    xg, wg = x.to(DEV), w.to(DEV)
    rg = res.to(DEV) if res is not None else None
    x_before = xg.clone()
    op.rms_norm_dynamic_per_token_quant_custom(out.t, xg, wg, sc.t, 1e-6, scale_ub.to(DEV) if scale_ub is not None else None, rg)
    torch.cuda.synchronize()
    out.check("codes"); sc.check("scales")
    assert torch.equal(xg, x_before), "input must not be modified"
    return out.t.cpu(), sc.t.cpu(), (rg.cpu() if rg is not None else None)


# shapes of the reference test (unit_test/test_fused_rms_norm_dq.py:17-22, token counts trimmed) + the benchmark shapes
SHAPES = [(1, 1), (1, 64), (1, 1024), (1, 1025), (1, 1026), (1, 1027), (1, 1028), (1, 1029), (1, 5120), (1, 5137),
          (83, 1), (83, 1033), (83, 2048), (83, 5120), (300, 64), (129, 5137), (256, 4096), (64, 7168), (48, 8192),
          (3, 16384), (2, 32768), (2, 40000), (40, 6144), (700, 4096), (333, 5120)]


@pytest.mark.parametrize("T,H", SHAPES)
@pytest.mark.parametrize("add_residual", [False, True])
def test_norm_quant_bf16_matches_oracle(op, T, H, add_residual):
    d = W.norm_quant_inputs(T, H)
    res = d["residual"] if add_residual else None
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(d["x"], d["weight"], 1e-6, residual=res)
    q, s, r = _run_a2(op, d["x"], d["weight"], res)
    C.assert_codes(q, q_ref, f"codes {T}x{H}")
    C.assert_close(s, s_ref, "scales")
    if add_residual:
        C.assert_equal(bits(r), bits(r_ref), "residual (bit-exact)")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("T,H", [(1, 64), (83, 1033), (17, 2048), (5, 5137)])
def test_norm_quant_other_dtypes(op, dtype, T, H):
    d = W.norm_quant_inputs(T, H, dtype=dtype)
    scale = 1.0 / H  # the reference test scales its inputs by 1/hidden
    x, res = (d["x"].float() * scale).to(dtype), (d["residual"].float() * scale).to(dtype)
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(x, d["weight"], 1e-6, residual=res)
    q, s, r = _run_a2(op, x, d["weight"], res)
    C.assert_codes(q, q_ref, f"codes {dtype}")
    C.assert_close(s, s_ref, "scales", abs_=1e-6)
    C.assert_equal(bits(r), bits(r_ref), "residual")


def test_norm_quant_against_golden(op, golden):
    """The reference's own test tolerances: allclose on scales, int8 atol=1, allclose on the residual."""
    n = 0
    for key, r in records(golden, "formula:unit_test/test_fused_rms_norm_dq.py:77-117"):
        q, s, res = _run_a2(op, r["x"], r["weight"], r.get("residual"))
        assert torch.allclose(s, r["scales"]), key
        assert C.code_stats(q, r["codes"])["max_abs"] <= 1, key
        if "residual_out" in r:
            assert torch.allclose(res.float(), r["residual_out"].float()), key
        n += 1
    assert n >= 20


def test_norm_quant_degenerate_rows(op):
    T, H = 8, 1024
    d = W.norm_quant_inputs(T, H)
    x, res = d["x"].clone(), d["residual"].clone()
    x[0] = 0; res[0] = 0                       # all-zero row: scale floors at FLT_EPSILON, codes are 0
    x[1] = 0; res[1] = 0; x[1, 5] = 3.0        # one-hot row
    x[2] = 60000.0; res[2] = 60000.0           # large values: the fp32 sum of squares must not overflow
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(x, d["weight"], 1e-6, residual=res)
    q, s, r = _run_a2(op, x, d["weight"], res)
    assert float(s[0]) == pytest.approx(FLT_EPSILON) and int(q[0].abs().max()) == 0
    C.assert_codes(q, q_ref); C.assert_close(s, s_ref, abs_=1e-7); C.assert_equal(bits(r), bits(r_ref))
    assert torch.isfinite(s).all()


def test_norm_quant_scale_ub(op):
    d = W.norm_quant_inputs(16, 2048)
    ub = torch.tensor([1.5])
    q_ref, s_ref, _ = R.rms_norm_dynamic_per_token_quant(d["x"], d["weight"], 1e-6, residual=d["residual"], scale_ub=ub)
    q, s, _ = _run_a2(op, d["x"], d["weight"], d["residual"], scale_ub=ub)
    assert float(s.max()) <= 1.5 / 127 + 1e-9
    C.assert_codes(q, q_ref); C.assert_close(s, s_ref)
    assert int(q.min()) == -128 or int(q.max()) == 127   # clamped values saturate


def test_norm_quant_is_deterministic(op):
    d = W.norm_quant_inputs(512, 7168)
    a = _run_a2(op, d["x"], d["weight"], d["residual"])
    b = _run_a2(op, d["x"], d["weight"], d["residual"])
    for u, v in zip(a, b):
        assert torch.equal(bits(u), bits(v))


def test_custom_ops_wrapper(op):
    from mcoplib_b200 import custom_ops
    d = W.norm_quant_inputs(32, 4096)
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(d["x"], d["weight"], 1e-6, residual=d["residual"])
    res = d["residual"].to(DEV)
    q, s = custom_ops.rms_norm_dynamic_per_token_quant(d["x"].to(DEV), d["weight"].to(DEV), 1e-6, torch.int8, None, res)
    assert q.dtype == torch.int8 and tuple(s.shape) == (32, 1) and s.dtype == torch.float32
    C.assert_codes(q, q_ref); C.assert_close(s, s_ref); C.assert_equal(bits(res), bits(r_ref))


def test_torch_library_ops(op):
    d = W.norm_quant_inputs(64, 4096)
    ns = getattr(torch.ops, op.torch_namespace)
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(d["x"], d["weight"], 1e-6, residual=d["residual"])
    out = torch.empty(64, 4096, dtype=torch.int8, device=DEV); sc = torch.empty(64, 1, device=DEV); res = d["residual"].to(DEV)
    ns.rms_norm_dynamic_per_token_quant(out, d["x"].to(DEV), d["weight"].to(DEV), sc, 1e-6, None, res)
    C.assert_codes(out, q_ref); C.assert_close(sc, s_ref); C.assert_equal(bits(res), bits(r_ref))
    o_ref, r2_ref = R.fused_add_rms_norm(d["x"], d["residual"], d["weight"], 1e-6)
    x, res = d["x"].to(DEV), d["residual"].to(DEV)
    ns.fused_add_rms_norm(x, res, d["weight"].to(DEV), 1e-6)
    C.assert_equal(bits(res), bits(r2_ref)); C.assert_close(x, o_ref)


@pytest.mark.parametrize("T,H", [(1, 8), (64, 4096), (7, 1030), (33, 8192), (5, 777),
                                 (1500, 7168), (1100, 8192), (2000, 4096), (1030, 1032), (1024, 5120), (1300, 16384)])  # >= 1024 rows: the pipelined kernel
def test_fused_add_rms_norm(op, T, H):
    d = W.norm_quant_inputs(T, H)
    o_ref, r_ref = R.fused_add_rms_norm(d["x"], d["residual"], d["weight"], 1e-6)
    x, res = d["x"].to(DEV), d["residual"].to(DEV)
    op.fused_add_rms_norm(x, res, d["weight"].to(DEV), 1e-6)
    C.assert_equal(bits(res), bits(r_ref), "residual"); C.assert_close(x, o_ref, "out")
    # at most a handful of bf16 roundings may flip through a 1-ulp difference of the row scalar
    assert int((bits(x) != bits(o_ref)).sum()) <= max(2, x.numel() // 2000)


def test_fused_add_rms_norm_pipelined_and_row_kernels_agree_bit_for_bit(op):
    """1500 rows go through the pipelined kernel, their first 1000 alone through the row-per-CTA kernel: same bits;
    also with a strided input."""
    d = W.norm_quant_inputs(1500, 7168)
    w = d["weight"].to(DEV)
    xa, ra = d["x"].to(DEV), d["residual"].to(DEV)
    op.fused_add_rms_norm(xa, ra, w, 1e-6)
    xb, rb = d["x"][:1000].to(DEV), d["residual"][:1000].to(DEV)
    op.fused_add_rms_norm(xb, rb, w, 1e-6)
    C.assert_equal(bits(xa[:1000]), bits(xb)); C.assert_equal(bits(ra[:1000]), bits(rb))
    big = torch.zeros(1500, 2 * 7168, dtype=torch.bfloat16, device=DEV)
    view = big[:, 7168:]
    view.copy_(d["x"])
    rc = d["residual"].to(DEV)
    op.fused_add_rms_norm(view, rc, w, 1e-6)
    C.assert_equal(bits(view), bits(xa)); C.assert_equal(bits(rc), bits(ra))
    assert float(big[:, :7168].abs().max()) == 0


def test_fused_add_rms_norm_strided_input(op):
    d = W.norm_quant_inputs(40, 2048)
    big = torch.zeros(40, 3 * 2048, dtype=torch.bfloat16, device=DEV)
    view = big[:, 2048:4096]
    view.copy_(d["x"])
    res = d["residual"].to(DEV)
    o_ref, r_ref = R.fused_add_rms_norm(d["x"], d["residual"], d["weight"], 1e-6)
    op.fused_add_rms_norm(view, res, d["weight"].to(DEV), 1e-6)
    C.assert_equal(bits(res), bits(r_ref)); C.assert_close(view, o_ref)
    assert float(big[:, :2048].abs().max()) == 0 and float(big[:, 4096:].abs().max()) == 0
    (key, g), = records(pytest.importorskip("tests.golden_io").load_golden(),
                        "formula:benchmark/runners/mcoplib_mxbenchmark_fused_add_rms_norm_runners.py:36-49")
    x, r = g["x"].to(DEV), g["residual"].to(DEV)
    op.fused_add_rms_norm(x, r, g["weight"].to(DEV), 1e-6)
    C.assert_equal(bits(r), bits(g["residual_out"]), key); C.assert_close(x, g["out"], key, rel=2e-2, abs_=2e-2)


@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T,H,with_res", [(16, 4096, True), (9, 1030, True), (16, 7168, False), (3, 333, False),
                                          (1100, 7168, True), (1300, 4096, False), (1024, 8192, True), (1200, 2056, False)])  # last four (bf16 weights): pipelined kernel
def test_fused_rms_norm_dq_nine_arguments(op, wdtype, T, H, with_res):
    """PARITY UNPINNED in the reference; checked against the restatement of op/fused_rms_norm_dq.cu:69-186."""
    d = W.norm_quant_inputs(T, H)
    g = torch.Generator().manual_seed(3)
    w = d["weight"].to(wdtype)
    smooth = (0.5 + torch.rand(H, generator=g)).to(wdtype)
    res = d["residual"] if with_res else None
    q_ref, s_ref, ar_ref, an_ref = R.fused_rms_norm_dq(d["x"], w, smooth, 1e-6, residual=res)
    out = torch.empty(T, H, dtype=torch.int8, device=DEV); sc = torch.empty(T, device=DEV)
    ar = torch.empty(T, H, dtype=torch.bfloat16, device=DEV); an = torch.empty_like(ar)
    op.rms_norm_dynamic_per_token_quant(out, d["x"].to(DEV), w.to(DEV), smooth.to(DEV), sc, 1e-6, ar, an,
                                        res.to(DEV) if with_res else None)
    C.assert_equal(bits(ar), bits(ar_ref), "after_res"); C.assert_close(an, an_ref, "after_norm")
    C.assert_close(sc.reshape(-1, 1), s_ref, "scales"); C.assert_codes(out, q_ref)


@pytest.mark.parametrize("with_res", [True, False])
def test_fused_rms_norm_dq_pipelined_and_row_kernels_agree_bit_for_bit(op, with_res):
    """1400 rows (pipelined kernel) against their first 900 alone (row-per-CTA kernel): every output has the same bits;
    an all-zero row gives scale 0 and codes 0 in both."""
    d = W.norm_quant_inputs(1400, 7168)
    x = d["x"].clone(); res = d["residual"].clone()
    x[5] = 0; res[5] = 0
    x, res, w = x.to(DEV), res.to(DEV), d["weight"].to(DEV)
    smooth = (0.5 + torch.rand(7168, generator=torch.Generator().manual_seed(3))).bfloat16().to(DEV)
    outs = []
    for n in (1400, 900):
        q = torch.empty(n, 7168, dtype=torch.int8, device=DEV); sc = torch.empty(n, device=DEV)
        ar = torch.empty(n, 7168, dtype=torch.bfloat16, device=DEV); an = torch.empty_like(ar)
        op.rms_norm_dynamic_per_token_quant(q, x[:n], w, smooth, sc, 1e-6, ar, an, res[:n] if with_res else None)
        outs.append((q, sc, ar, an))
    (qa, sa, ara, ana), (qb, sb, arb, anb) = outs
    C.assert_equal(qa[:900], qb); C.assert_equal(bits(ara[:900]), bits(arb)); C.assert_equal(bits(ana[:900]), bits(anb))
    assert torch.equal(sa[:900].view(torch.int32), sb.view(torch.int32))
    assert float(sa[5]) == 0.0 and int(qa[5].abs().max()) == 0


@pytest.mark.parametrize("rms_div", [False, True])
@pytest.mark.parametrize("T,H,with_res", [(8, 1024, True), (5, 4096, False), (4, 999, True),
                                          (1100, 7168, True), (1500, 4096, False), (1024, 8192, True), (1200, 2056, False)])  # last four: pipelined kernel
def test_rms_norm(op, rms_div, T, H, with_res, golden):
    d = W.norm_quant_inputs(T, H)
    res = d["residual"] if with_res else None
    o_ref, ar_ref = R.rms_norm(d["x"], d["weight"], 1e-6, residual=res, rms_div=rms_div)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    ar = torch.empty_like(out) if with_res else None
    op.rms_norm(out, d["x"].to(DEV), d["weight"].to(DEV), 1e-6, ar, res.to(DEV) if with_res else None, rms_div)
    C.assert_close(out, o_ref)
    if with_res:
        C.assert_equal(bits(ar), bits(ar_ref))
    if rms_div and with_res and H == 1024:
        (key, g), = records(golden, "ref:unit_test/test_rms_norm.py:rms_norm_ref")
        out = torch.empty(8, 1024, dtype=torch.bfloat16, device=DEV); ar = torch.empty_like(out)
        op.rms_norm(out, g["x"].to(DEV), g["weight"].to(DEV), 1e-6, ar, g["residual"].to(DEV), True)
        C.assert_close(out, g["out"], key, rel=2e-2, abs_=2e-2)


@pytest.mark.parametrize("rms_div", [False, True])
def test_rms_norm_pipelined_and_row_kernels_agree_bit_for_bit(op, rms_div):
    """1400 rows (pipelined kernel) against their first 900 alone (row-per-CTA kernel); with a residual and its
    after_res output, and without a residual."""
    d = W.norm_quant_inputs(1400, 7168)
    x, res, w = d["x"].to(DEV), d["residual"].to(DEV), d["weight"].to(DEV)
    for with_res, with_ar in ((True, True), (False, False)):  # the shim wants residual and after_res together
        oa = torch.empty(1400, 7168, dtype=torch.bfloat16, device=DEV); ob = torch.empty(900, 7168, dtype=torch.bfloat16, device=DEV)
        ara = torch.empty_like(oa) if with_ar else None
        arb = torch.empty_like(ob) if with_ar else None
        op.rms_norm(oa, x, w, 1e-6, ara, res if with_res else None, rms_div)
        op.rms_norm(ob, x[:900], w, 1e-6, arb, res[:900] if with_res else None, rms_div)
        C.assert_equal(bits(oa[:900]), bits(ob))
        if with_ar:
            C.assert_equal(bits(ara[:900]), bits(arb))
    assert torch.equal(bits(x), bits(d["x"].to(DEV))) and torch.equal(bits(res), bits(d["residual"].to(DEV)))  # inputs untouched


def test_head_rms_norm_and_scale_dynamic_quant(op, golden):
    (key, g), = records(golden, "ref:unit_test/test_head_rms_norm.py:head_rms_norm_ref")
    hid = g["hidden"].to(DEV)
    out = hid.clone()
    op.head_rms_norm(out, hid, g["weight"].to(DEV), 1e-5, 0, g["head_norm"])
    ref = R.head_rms_norm(g["hidden"], g["weight"], 1e-5, 0, g["head_norm"])
    C.assert_close(out, ref, key); C.assert_close(out, g["out"], key, rel=2e-2, abs_=2e-2)
    for key, g in records(golden, "ref:unit_test/test_scale_dynamic_quant.py:scale_dynamic_quant_cpu"):
        q, s = op.scale_dynamic_quant(g["hidden"].to(DEV), g["smooth"].to(DEV))
        assert q.shape == g["hidden"].shape and s.numel() == g["scales"].numel()
        assert torch.allclose(s.cpu(), g["scales"].reshape(-1), rtol=1e-5), key
        assert C.code_stats(q.cpu(), g["codes"])["max_abs"] <= 1, key


def test_norm_quant_full_size_properties(op):
    """Benchmark configuration 4 (32768 x 8192): size-independent properties on the whole output, and the oracle
    on a sample of rows."""
    T, H = 32768, 8192
    d = W.norm_quant_inputs(T, H, gen_device=DEV)
    x, res, w = d["x"], d["residual"], d["weight"]
    res0 = res.clone()
    codes = torch.empty(T, H, dtype=torch.int8, device=DEV); sc = torch.empty(T, 1, device=DEV)
    op.rms_norm_dynamic_per_token_quant_custom(codes, x, w, sc, 1e-6, None, res)
    # residual == bf16(x + residual) exactly
    assert torch.equal(res, (x.float() + res0.float()).bfloat16())
    # every row uses the full code range: its abs-max element maps to +-127, nothing beyond
    amax = codes.to(torch.int16).abs().amax(dim=1)
    assert int(amax.min()) == 127 and int(amax.max()) == 127
    # scale * 127 equals the abs-max of the normalised row (checked with torch on the GPU in fp32)
    s = x.float() + res0.float()
    n = ((s * torch.rsqrt((s * s).mean(-1, keepdim=True) + 1e-6)).bfloat16() * w).float()
    assert torch.allclose(sc * 127.0, n.abs().amax(-1, keepdim=True), rtol=1e-2, atol=1e-3)
    # dequantised codes reproduce the normalised row to half a code
    # (torch's approximate rsqrt may flip either bf16 rounding of n: up to two bf16 ulps, 2^-6 relative)
    assert bool(((codes.float() * sc - n).abs() <= 0.51 * sc + 0.02 * n.abs()).all())
    # oracle on 256 sampled rows
    idx = torch.arange(0, T, T // 256, device=DEV)
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(x[idx].cpu(), w.cpu(), 1e-6, residual=res0[idx].cpu())
    C.assert_codes(codes[idx], q_ref); C.assert_close(sc[idx], s_ref); C.assert_equal(bits(res[idx]), bits(r_ref))


def test_c_abi_called_directly(op):
    """One call through ctypes with raw pointers: the binding a non-torch host would use."""
    from mcoplib_b200 import cabi
    from tests.gpu_util import stream_ptr
    lib = cabi.load()
    d = W.norm_quant_inputs(96, 4096)
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(d["x"], d["weight"], 1e-6, residual=d["residual"])
    x, w, res = d["x"].to(DEV), d["weight"].to(DEV), d["residual"].to(DEV)
    out = torch.empty(96, 4096, dtype=torch.int8, device=DEV); sc = torch.empty(96, device=DEV)
    rc = lib.mcop_add_rmsnorm_quant_i8(out.data_ptr(), sc.data_ptr(), x.data_ptr(), 4096, w.data_ptr(), res.data_ptr(), None,
                                       96, 4096, 1e-6, cabi.BF16_CODE, stream_ptr())
    cabi.check(rc, lib)
    torch.cuda.synchronize()
    C.assert_codes(out, q_ref); C.assert_close(sc.reshape(-1, 1), s_ref); C.assert_equal(bits(res), bits(r_ref))
    # a misaligned row stride falls back to the scalar kernel and still matches
    xs = torch.zeros(96, 4099, dtype=torch.bfloat16, device=DEV)
    xs[:, :4096] = d["x"].to(DEV)
    res = d["residual"].to(DEV)
    rc = lib.mcop_add_rmsnorm_quant_i8(out.data_ptr(), sc.data_ptr(), xs.data_ptr(), 4099, w.data_ptr(), res.data_ptr(), None,
                                       96, 4096, 1e-6, cabi.BF16_CODE, stream_ptr())
    cabi.check(rc, lib)
    torch.cuda.synchronize()
    C.assert_codes(out, q_ref); C.assert_equal(bits(res), bits(r_ref))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_dynamic_scaled_int8_quant(op, dtype):
    ns = getattr(torch.ops, op.torch_namespace)
    x = W.per_token("randn", 60, 0, 130, 4100, dtype)
    x[7] = 0
    q_ref, s_ref = R.dynamic_scaled_int8_quant(x)
    out = Canary((130, 4100), torch.int8); sc = Canary((130, 1), torch.float32)
    ns.dynamic_scaled_int8_quant(out.t, x.to(DEV), sc.t, None)
    torch.cuda.synchronize()
    out.check(); sc.check()
    C.assert_codes(out.t, q_ref); C.assert_close(sc.t, s_ref, abs_=1e-7)
    assert int(out.t[7].abs().max()) == 0
    with pytest.raises(RuntimeError):
        ns.dynamic_scaled_int8_quant(out.t, x.to(DEV), sc.t, torch.zeros(130, 1, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T,H", [(3000, 7168), (500, 4096), (64, 520), (33, 100)])
def test_scale_dynamic_quant_is_exact_on_wide_ranges(op, dtype, T, H):
    """The vector kernel (row in registers, x and smooth read once) against the oracle, bit for bit: rows spread over
    40 binades (f16 rows overflow to infinity there: codes 0 like the oracle's), an all-zero row."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g) * torch.exp2(torch.randint(-20, 20, (T, 1), generator=g).float())
    x[7] = 0
    x = x.to(dtype)
    smooth = 0.25 + 2 * torch.rand(H, generator=g)
    q_ref, s_ref = R.scale_dynamic_quant(x, smooth)
    q, s = op.scale_dynamic_quant(x.to(DEV), smooth.to(DEV))
    C.assert_equal(bits(s.cpu()), bits(s_ref.reshape(-1)), "scales")
    C.assert_equal(q.cpu(), q_ref, "codes")
    assert int(q[7].abs().max()) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,H", [(2048, 4096), (1100, 8192), (1024, 2056), (4000, 7168), (1500, 5120)])
def test_scale_dynamic_quant_pipelined_shapes_ties_and_special_rows(op, dtype, T, H):
    """From 1024 rows of 2048 .. 16384 two-byte elements the persistent, pipelined kernel takes over.  It forms y / scale
    as y * (1 / scale) and falls back to the division near a tie, so the cases are: random rows over 40 binades, rows of
    small integers whose scale is exactly 2 (every other code is an exact tie k + 0.5: round half to even), a row with an
    infinity, an all-zero row, a row so small that 1 / scale overflows - all bit for bit."""
    g = torch.Generator().manual_seed(21)
    x = torch.randn(T, H, generator=g) * torch.exp2(torch.randint(-20, 20, (T, 1), generator=g).float())
    ties = torch.randint(-254, 255, (64, H), generator=g).float()
    ties[:, 0] = 254.0                      # scale = 254 / 127 = 2 exactly
    x[100:164] = ties
    x[5] = 0
    x[11, 17] = float("inf")
    x[13] = torch.randn(H, generator=g) * 1e-38
    x = x.to(dtype)
    smooth = 0.25 + 2 * torch.rand(H, generator=g)
    smooth_one = torch.ones(H)
    for sm in (smooth, smooth_one):
        q_ref, s_ref = R.scale_dynamic_quant(x, sm)
        q, s = op.scale_dynamic_quant(x.to(DEV), sm.to(DEV))
        assert _device_error_word() == 0
        C.assert_equal(bits(s.cpu()), bits(s_ref.reshape(-1)), "scales")
        C.assert_equal(q.cpu(), q_ref, "codes")
    assert int((q_ref[100:164].abs() == 127).sum()) >= 64  # the tie rows really are scaled by 2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,H", [(2048, 4096), (1100, 8192), (1024, 2056), (4000, 7168)])
def test_dynamic_scaled_int8_quant_pipelined_shapes(op, dtype, T, H):
    """The same persistent kernel without the smooth vector (torch.ops._C.dynamic_scaled_int8_quant, symmetric form)."""
    ns = getattr(torch.ops, op.torch_namespace)
    g = torch.Generator().manual_seed(22)
    x = (torch.randn(T, H, generator=g) * torch.exp2(torch.randint(-12, 12, (T, 1), generator=g).float()))
    x[7] = 0
    x = x.to(dtype)
    q_ref, s_ref = R.dynamic_scaled_int8_quant(x)
    out = Canary((T, H), torch.int8); sc = Canary((T, 1), torch.float32)
    ns.dynamic_scaled_int8_quant(out.t, x.to(DEV), sc.t, None)
    torch.cuda.synchronize()
    out.check(); sc.check()
    assert _device_error_word() == 0
    C.assert_equal(out.t.cpu(), q_ref, "codes"); C.assert_equal(bits(sc.t.cpu()), bits(s_ref), "scales")
    assert int(out.t[7].abs().max()) == 0


@pytest.mark.parametrize("dtype,wdtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32), (torch.float32, torch.float32)])
@pytest.mark.parametrize("D", [64, 128, 256, 80])
def test_head_rms_norm_vector_kernel_is_exact(op, dtype, wdtype, D):
    """Heads of 64, 128 and 256 elements take the 16-byte kernel (80 stays on the element kernel): the oracle's
    x / r * w to the last bit on all but a handful of elements (the CPU's and the GPU's sqrt / division chain may differ
    by an fp32 ulp, which can move a 16-bit rounding), heads outside [head_offset, head_offset + head_norm) untouched."""
    T, heads = 700, 12
    g = torch.Generator().manual_seed(12)
    x = (torch.randn(T, heads, D, generator=g) * torch.exp2(torch.randint(-8, 8, (T, heads, 1), generator=g).float())).to(dtype)
    w = (1 + 0.1 * torch.randn(heads, D, generator=g)).to(wdtype)
    ref = R.head_rms_norm(x, w, 1e-5, 3, 7)
    out = torch.full_like(x, 9.0).to(DEV)
    op.head_rms_norm(out, x.to(DEV), w.to(DEV), 1e-5, 3, 7)
    got, want = out[:, 3:10].cpu(), ref[:, 3:10]
    C.assert_close(got, want, "normalised heads", rel=1e-2 if dtype != torch.float32 else 1e-6, abs_=1e-6)
    if dtype != torch.float32:   # (in fp32 the ulp of the scalar r shows directly: the tolerance above is the check)
        assert int((bits(got) != bits(want)).sum()) <= max(3, got.numel() // 100000), "more than a few last-bit differences"
    assert bool((out[:, :3] == 9).all()) and bool((out[:, 10:] == 9).all())


@pytest.mark.parametrize("dtype,wdtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16), (torch.float32, torch.float32)])
@pytest.mark.parametrize("T,heads,D,off,hn", [(9000, 12, 128, 3, 7), (20000, 8, 64, 0, 8), (5000, 5, 256, 1, 3),
                                              (3000, 40, 128, 4, 32), (2000, 70, 64, 0, 70), (1500, 20, 256, 2, 17), (1200, 56, 128, 0, 56)])
def test_head_rms_norm_grid_stride_and_corrected_quotients(op, dtype, wdtype, T, heads, D, off, hn):
    """Both pipelined forms (one and four vectors per lane: the latter from 25 heads of 128 to normalise), more heads than
    one turn of the grid holds (the walk's add-and-carry of token and head), and the value ranges the
    quotient correction has to treat apart: heads spread over 60 binades, a head of zeros, a head whose nonzero values sit
    below 2^-60 (they take the division itself).  Against the oracle: a handful of last-bit
    differences at most in 16-bit outputs (the scalar r may differ by an fp32 ulp between CPU and GPU), 1e-6 in fp32."""
    g = torch.Generator().manual_seed(31)
    lo, hi = (-30, 30) if dtype != torch.float16 else (-10, 6)
    x = torch.randn(T, heads, D, generator=g) * torch.exp2(torch.randint(lo, hi, (T, heads, 1), generator=g).float())
    x[3, off] = 0
    x[4, off] = 0
    if dtype != torch.float16:
        x[4, off, 5] = 2.0 ** -70
        x[5, off + hn - 1] = torch.randn(D, generator=g) * 2.0 ** -75
    x = x.to(dtype)
    w = (1 + 0.1 * torch.randn(heads, D, generator=g)).to(wdtype)
    ref = R.head_rms_norm(x, w, 1e-5, off, hn)
    out = torch.full_like(x, 9.0).to(DEV)
    op.head_rms_norm(out, x.to(DEV), w.to(DEV), 1e-5, off, hn)
    got, want = out[:, off:off + hn].cpu(), ref[:, off:off + hn]
    assert bool(torch.isfinite(got.float()).all())
    if dtype == torch.float32:
        C.assert_close(got, want, "normalised heads", rel=1e-6, abs_=1e-30)
    else:
        diff = bits(got) != bits(want)
        assert int(diff.sum()) <= max(3, got.numel() // 100000), f"{int(diff.sum())} last-bit differences"
        C.assert_close(got, want, "normalised heads", rel=1e-2, abs_=1e-30)
    assert bool((out[:, :off] == 9).all()) and bool((out[:, off + hn:] == 9).all())
    # in place, as the reference's callers use it
    xin = x.to(DEV)
    op.head_rms_norm(xin, xin, w.to(DEV), 1e-5, off, hn)
    assert torch.equal(bits(xin[:, off:off + hn]), bits(out[:, off:off + hn]))


def test_scale_dynamic_quant_adversarial_ties_fp32(op):
    """The division-free code path against the IEEE division on inputs built to sit on and beside the rounding ties: for a
    set of scales (random ones, and mantissas of all zeros, all ones, a single low or high bit), a row holds 127 * scale as
    its maximum and, for every k, the fp32 value nearest to scale * (k + 0.5) with its neighbours one and two ulps either
    side, in both signs.  fp32 rows with a smooth vector of ones (y = x exactly): the row-per-CTA kernel, which shares
    `quant8_by_scale` with the pipelined one.  Bit-exact codes and scales."""
    import numpy as np
    rng = np.random.default_rng(3)
    mant = np.concatenate([rng.integers(0, 1 << 23, 200), [0, 0x7fffff, 1, 0x400000, 0x7ffffe, 0x2aaaaa, 0x555555]]).astype(np.uint32)
    expo = rng.integers(100, 150, mant.size).astype(np.uint32)
    scales = ((expo << 23) | mant).view(np.float32)
    H = 2048
    rows = []
    for sc in scales:
        top = np.float32(127.0) * sc
        k = np.arange(0, 127, dtype=np.float32) + np.float32(0.5)
        base = (k * sc).astype(np.float32)
        vals = [base]
        for d in (1, 2):
            up, dn = base.copy(), base.copy()
            for _ in range(d):
                up = np.nextafter(up, np.float32(np.inf)); dn = np.nextafter(dn, np.float32(0))
            vals += [up, dn]
        v = np.concatenate(vals)
        v = np.concatenate([v, -v])
        row = np.zeros(H, np.float32)
        row[0] = top
        row[1:1 + v.size] = v[: H - 1]
        rows.append(row)
    x = torch.from_numpy(np.stack(rows))
    assert bool(torch.isfinite(x).all())
    ones = torch.ones(H)
    q_ref, s_ref = R.scale_dynamic_quant(x, ones)
    q, s = op.scale_dynamic_quant(x.to(DEV), ones.to(DEV))
    C.assert_equal(bits(s.cpu()), bits(s_ref.reshape(-1)), "scales")
    C.assert_equal(q.cpu(), q_ref, "codes")
    # the same rows as bf16-representable values through the pipelined kernel (rows repeated to reach its 1024-row threshold)
    xb = x.bfloat16().repeat(6, 1)
    q_ref, s_ref = R.scale_dynamic_quant(xb, ones)
    q, s = op.scale_dynamic_quant(xb.to(DEV), ones.to(DEV))
    C.assert_equal(bits(s.cpu()), bits(s_ref.reshape(-1)), "scales (bf16 rows)")
    C.assert_equal(q.cpu(), q_ref, "codes (bf16 rows)")


@pytest.mark.parametrize("T,heads,D", [(2000, 56, 128), (1500, 16, 64), (300, 12, 256)])
def test_head_rms_norm_quotients_against_ieee_division_fp32(op, T, heads, D):
    """The twice-corrected quotient x * (1 / r) of the head kernels against the IEEE division, bit for bit, on fp32 heads
    (no rounding to a 16-bit type hides a last-bit error): the checker is torch on the GPU with the same formula -
    the mean of squares in float64 rounded to fp32, r = 1 / sqrt(var + eps), (x / r) * w - whose sqrt and divisions are the
    IEEE ones.  Heads spread over 40 binades; both the pipelined kernel (T >= 1024) and the grid-stride kernel."""
    g = torch.Generator(device=DEV).manual_seed(41)
    x = torch.randn(T, heads, D, generator=g, device=DEV) * torch.exp2(torch.randint(-20, 20, (T, heads, 1), generator=g, device=DEV).float())
    w = 1 + 0.1 * torch.randn(heads, D, generator=g, device=DEV)
    var = (x.double() * x.double()).mean(dim=-1, keepdim=True).float()
    r = 1.0 / torch.sqrt(var + 1e-5)
    ref = (x / r) * w.unsqueeze(0)
    out = torch.empty_like(x)
    op.head_rms_norm(out, x, w, 1e-5, 0, heads)
    assert torch.equal(bits(out), bits(ref)), f"{int((bits(out) != bits(ref)).sum())} of {out.numel()} elements differ"
