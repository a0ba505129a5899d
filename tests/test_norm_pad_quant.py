"""fused_add_rms_norm_dynamic_per_token_quant_padding_output: residual add + RMSNorm + int8 quantisation with a padded
record per token (codes, then the fp32 scale).  The reference test of this operator asserts nothing, so parity is
the oracle's restatement of the two kernels the reference selects by row length; codes are compared bit for bit
up to the +-1 LSB allowance on <= 0.01 % of elements, scales and the bf16 norm output exactly up to 1e-6 / 1 ulp."""
import pytest
import torch

from mcoplib_b200 import workloads as W
from oracle import compare as C
from oracle import ref_ops as R


def _inputs(T, H, dtype=torch.bfloat16, seed=0):
    d = W.norm_quant_inputs(T, H, seed=seed)
    return d["x"].to(dtype), d["residual"].to(dtype), d["weight"].to(dtype)


def test_oracle_forms_and_record_layout():
    x, res, w = _inputs(6, 64)
    packed, new_res, norm, q, sc = R.fused_add_rms_norm_dynamic_per_token_quant_padding_output(x, res, w, 40, 1e-6)
    assert packed.shape == (6, 80) and q.shape == (6, 64) and sc.shape == (6, 1)
    assert torch.equal(packed[:, :64].contiguous().view(torch.int8), q)
    assert torch.equal(packed[:, 64:68].contiguous().view(torch.float32).reshape(-1), sc.reshape(-1))
    assert int(packed[:, 68:].max()) == 0
    assert torch.equal(new_res, (x.float() + res.float()).to(torch.bfloat16))
    # the default form follows the row length: 2 unless the row has 7168 elements
    p2 = R.fused_add_rms_norm_dynamic_per_token_quant_padding_output(x, res, w, 40, 1e-6, form=2)[0]
    assert torch.equal(packed, p2)
    # form 2's norm output is fused_add_rms_norm's up to the variance taken from the unrounded sum (rare 1-ulp flips),
    # and dequantised codes approximate it
    n_ref, _ = R.fused_add_rms_norm(x, res, w, 1e-6)
    assert float((norm.float() != n_ref.float()).float().mean()) < 0.1
    assert torch.allclose(norm.float(), n_ref.float(), rtol=2 ** -6, atol=1e-6)
    assert float((q.float() * sc - norm.float()).abs().max()) <= float(sc.max()) * 0.51 + 1e-6
    # form 1 differs only by where it rounds
    _, _, norm1, q1, sc1 = R.fused_add_rms_norm_dynamic_per_token_quant_padding_output(x, res, w, 40, 1e-6, form=1)
    assert float((norm1.float() - norm.float()).abs().max()) <= 0.05 and int((q1.int() - q.int()).abs().max()) <= 2


@pytest.mark.gpu
@pytest.mark.parametrize("T,H,pad", [(5, 7168, 3840), (67, 4096, 2304), (33, 1024, 514), (9, 100, 64), (3, 8192, 4352),
                                      (2, 16384, 8448)])
def test_operator_matches_oracle(T, H, pad):
    from mcoplib_b200 import custom_ops
    from tests.gpu_util import DEV
    x, res, w = _inputs(T, H)
    x[1] = 0; res[1] = 0                                    # an all-zero row: scale floors at FLT_EPSILON, codes 0
    p_ref, r_ref, n_ref, q_ref, s_ref = R.fused_add_rms_norm_dynamic_per_token_quant_padding_output(x, res, w, pad, 1e-6)
    xd, rd, wd = x.to(DEV), res.to(DEV).clone(), w.to(DEV)
    out, res_out, out_rms, out_q, scales = custom_ops.fused_add_rms_norm_dynamic_per_token_quant_padding_output(xd, rd, wd, pad, 1e-6)
    assert out.shape == (T, pad) and out.dtype == torch.bfloat16 and res_out.data_ptr() == rd.data_ptr()
    rec = out.cpu().view(torch.uint8).reshape(T, 2 * pad)
    C.assert_codes(rec[:, :H].contiguous().view(torch.int8), q_ref, "packed codes")
    C.assert_codes(out_q, q_ref, "plain codes")
    C.assert_close(rec[:, H:H + 4].contiguous().view(torch.float32).reshape(-1), s_ref.reshape(-1), "packed scale", rel=1e-6, abs_=0)
    C.assert_close(scales.reshape(-1), s_ref.reshape(-1), "scales", rel=1e-6, abs_=0)
    assert torch.equal(res_out.cpu(), r_ref)
    C.assert_close(out_rms.float(), n_ref.float(), "norm output", rel=2 ** -6, abs_=1e-6)   # one bf16 ulp
    assert float((out_rms.cpu().float() != n_ref.float()).float().mean()) < 1e-3
    assert torch.equal(torch.from_numpy(rec.numpy()[1, :H]).view(torch.int8), torch.zeros(H, dtype=torch.int8))


@pytest.mark.gpu
@pytest.mark.parametrize("H,form,dtype", [(1024, 1, torch.bfloat16), (7168, 2, torch.bfloat16), (520, 1, torch.float16),
                                          (2048, 2, torch.float16)])
def test_c_abi_with_an_explicit_form_leaves_the_padding_alone(H, form, dtype):
    from mcoplib_b200 import cabi
    from tests.gpu_util import DEV, stream_ptr
    T, pad = 11, H // 2 + 64
    x, res, w = _inputs(T, H, dtype, seed=2)
    p_ref, r_ref, n_ref, q_ref, s_ref = R.fused_add_rms_norm_dynamic_per_token_quant_padding_output(x, res, w, pad, 1e-5, form=form)
    xd, rd, wd = x.to(DEV), res.to(DEV), w.to(DEV)
    packed = torch.full((T, 2 * pad), 0x5A, dtype=torch.uint8, device=DEV)
    lib = cabi.load()
    code = cabi.BF16_CODE if dtype == torch.bfloat16 else cabi.F16_CODE
    rc = lib.mcop_add_rmsnorm_quant_i8_padded(xd.data_ptr(), rd.data_ptr(), wd.data_ptr(), packed.data_ptr(), None, None, None,
                                              T, H, pad, 1e-5, form, code, stream_ptr())
    cabi.check(rc, lib)
    torch.cuda.synchronize()
    rec = packed.cpu()
    C.assert_codes(rec[:, :H].contiguous().view(torch.int8), q_ref)
    C.assert_close(rec[:, H:H + 4].contiguous().view(torch.float32).reshape(-1), s_ref.reshape(-1), rel=1e-6, abs_=0)
    assert bool((rec[:, H + 4:] == 0x5A).all())
    assert torch.equal(rd.cpu(), r_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("T,H,dtype,with_res", [(300, 7168, torch.bfloat16, True), (64, 8192, torch.bfloat16, True),
                                                (40, 4096, torch.bfloat16, False), (17, 1000, torch.float16, True),
                                                (5, 36, torch.bfloat16, True), (20000, 7168, torch.bfloat16, True)])
def test_sglang_flavour_also_returns_the_normalised_row(T, H, dtype, with_res):
    """rms_norm_dynamic_per_token_quant_custom(out, out_bf16, ...) of sglang: same codes / scales / residual as the
    7-argument operator, bit for bit, plus n (every size class: pipelined, row-per-CTA, unaligned)."""
    from mcoplib_b200 import op
    from tests.gpu_util import DEV, Canary, bits
    x, res, w = _inputs(T, H, dtype, seed=4)
    xd, wd = x.to(DEV), w.to(DEV)
    r1 = res.to(DEV) if with_res else None
    r2 = res.to(DEV) if with_res else None
    q1 = torch.empty(T, H, dtype=torch.int8, device=DEV); s1 = torch.empty(T, 1, device=DEV)
    op.rms_norm_dynamic_per_token_quant_custom(q1, xd, wd, s1, 1e-6, None, r1)
    q2 = Canary((T, H), torch.int8); n2 = Canary((T, H), dtype); s2 = torch.empty(T, 1, device=DEV)
    op.sgl_rms_norm_dynamic_per_token_quant_custom(q2.t, n2.t, xd, wd, s2, 1e-6, None, r2)
    torch.cuda.synchronize()
    q2.check(); n2.check()
    assert torch.equal(q1, q2.t) and torch.equal(s1, s2)
    if with_res:
        assert torch.equal(bits(r1), bits(r2))
    if T <= 1000:
        q_ref, s_ref, _, n_ref = R.rms_norm_dynamic_per_token_quant(x, w, 1e-6, residual=res if with_res else None, return_norm=True)
        C.assert_codes(q2.t, q_ref)
        assert float((n2.t.cpu().float() != n_ref.float()).float().mean()) < 1e-4
        C.assert_close(n2.t.float(), n_ref.float(), "norm output", rel=2 ** -6, abs_=1e-6)
    else:   # size-independent property: the codes are the quantised normalised row
        back = torch.round(n2.t.cpu().float() * (1.0 / s2.cpu())).clamp(-128, 127).to(torch.int8)
        assert torch.equal(back, q2.t.cpu())
    with pytest.raises(RuntimeError):
        op.sgl_rms_norm_dynamic_per_token_quant_custom(q2.t, n2.t, xd, wd, s2, 1e-6, torch.ones(1, device=DEV), r2)


@pytest.mark.gpu
def test_rejects_a_record_too_small_and_wrong_dtypes():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    x, res, w = (t.to(DEV) for t in _inputs(4, 256))
    good = dict(out=torch.empty(4, 2 * 160, dtype=torch.int8, device=DEV), rms=torch.empty_like(x),
                q=torch.empty(4, 256, dtype=torch.int8, device=DEV), sc=torch.empty(4, 1, device=DEV))
    op.fused_add_rms_norm_dynamic_per_token_quant_padding_output(good["out"], good["rms"], good["q"], good["sc"], x, res.clone(), w, 160, 1e-6)
    with pytest.raises(RuntimeError):   # 2 * 129 bytes cannot hold 256 codes + 4
        op.fused_add_rms_norm_dynamic_per_token_quant_padding_output(torch.empty(4, 258, dtype=torch.int8, device=DEV), good["rms"],
                                                                     good["q"], good["sc"], x, res.clone(), w, 129, 1e-6)
    with pytest.raises(RuntimeError):   # fp16 input: the reference accepts bf16 only
        op.fused_add_rms_norm_dynamic_per_token_quant_padding_output(good["out"], good["rms"].half(), good["q"], good["sc"], x.half(),
                                                                     res.half(), w.half(), 160, 1e-6)
