"""fused_silu_mul_dq_reorder_quant / fused_silu_mul_dq_mask_quant / fused_silu_mul_dq_quant (SiLU(gate)*up followed by
per-row int8 quantisation): the oracle against the golden vector made by the reference test's own torch quantiser,
and the CUDA kernels against the oracle (codes +-1 LSB on <= 0.01 %: CPU exp and CUDA expf differ in the last ulp;
scales 1e-5 relative).  Rows the operators must not process are checked to stay untouched."""
import pytest
import torch

from mcoplib_b200 import workloads as W
from oracle import compare as C
from oracle import ref_ops as R
from tests.golden_io import records


def test_oracle_row_quant_matches_reference_torch_function(golden):
    (key, r), = records(golden, "ref:unit_test/test_silu_mul_dq_reorder_mask.py:ref_dynamic_per_token_quant")
    v = R.silu_mul(r["gate_up"])
    assert torch.equal(v, r["product"]), key
    q, s = R.absmax_row_quant(v)
    assert C.code_stats(q, r["codes"])["max_abs"] <= 1, key
    assert C.code_stats(q, r["codes"])["frac_diff"] < 1e-3, key
    assert torch.allclose(s, r["scales"], rtol=1e-6), key


def test_oracle_reorder_and_mask_forms_agree_on_processed_rows():
    x = W.per_token("randn", 71, 0, 24, 2 * 64, torch.bfloat16, seed=3)[:24]
    ids = torch.tensor([0, 5, 2, 9, 3, 3, 7, 1] * 3, dtype=torch.int64)
    q, s, act = R.fused_silu_mul_dq_reorder_quant(x, ids, 1, 5)
    assert act.tolist() == [(1 <= int(i) <= 5) for i in ids]
    assert int(q[~act].abs().max()) == 0 and float(s[~act].abs().max()) == 0.0
    packed, written = R.fused_silu_mul_dq_mask_quant(x.reshape(2, 12, 128), torch.tensor([5, 12]))
    assert packed.shape == (2, 12, R.silu_mul_pack_stride(128) * 2) and R.silu_mul_pack_stride(128) == 256
    qa, sa, _ = R.fused_silu_mul_dq_reorder_quant(x, None, 0, 0)
    pk = packed.reshape(24, -1)
    w = written.reshape(-1)
    assert w.tolist() == [m < 5 for m in range(12)] + [True] * 12
    assert torch.equal(pk[w][:, :64].contiguous().view(torch.int8), qa[w])
    assert torch.equal(pk[w][:, 64:68].contiguous().view(torch.float32).reshape(-1), sa[w])
    assert int(pk[~w].max()) == 0


def _x(rows, n, dtype, seed=0):
    return W.per_token("randn", 72, 0, max(rows, 1), 2 * n, dtype, seed=seed)[:rows]


@pytest.mark.gpu
@pytest.mark.parametrize("rows,n,dtype,idt", [(37, 256, torch.bfloat16, torch.int64), (300, 2048, torch.bfloat16, torch.int32),
                                              (64, 7168, torch.float16, torch.int64), (9, 100, torch.bfloat16, torch.int32),
                                              (12, 16384, torch.bfloat16, torch.int64), (5, 36, torch.float16, torch.int32),
                                              (131, 1024, torch.float16, torch.int64), (3, 2048, torch.float16, torch.int32)])
def test_reorder_quant_matches_oracle(rows, n, dtype, idt):
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    x = _x(rows, n, dtype)
    x[1] = 0                                              # an all-zero row: codes 0, scale 0
    ids = torch.randint(0, 12, (rows,), generator=torch.Generator().manual_seed(rows), dtype=idt)
    ids[1] = 4
    q_ref, s_ref, act = R.fused_silu_mul_dq_reorder_quant(x, ids, 2, 8)
    out = torch.full((rows, n), 7, dtype=torch.int8, device=DEV)
    sc = torch.full((rows, 1), -1.0, device=DEV)
    op.fused_silu_mul_dq_reorder_quant(out, sc, x.to(DEV), ids.to(DEV), torch.empty(0), 2, 8)
    out, sc = out.cpu(), sc.cpu().reshape(-1)
    C.assert_codes(out[act], q_ref[act]); C.assert_close(sc[act], s_ref[act], rel=1e-5, abs_=1e-9)
    assert bool((out[~act] == 7).all()) and bool((sc[~act] == -1.0).all())
    assert int(out[1].abs().max()) == 0 and float(sc[1]) == 0.0


@pytest.mark.gpu
def test_unmasked_form_processes_every_row():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV, Canary
    x = _x(50, 1536, torch.bfloat16, seed=2)
    q_ref, s_ref, _ = R.fused_silu_mul_dq_reorder_quant(x, None, 0, 0)
    out = Canary((50, 1536), torch.int8); sc = Canary((50,), torch.float32)
    op.fused_silu_mul_dq_quant(out.t, sc.t, x.to(DEV))
    torch.cuda.synchronize()
    out.check(); sc.check()
    C.assert_codes(out.t, q_ref); C.assert_close(sc.t, s_ref, rel=1e-5, abs_=1e-9)


@pytest.mark.gpu
@pytest.mark.parametrize("G,M,n,counts,dtype,mdt", [(2, 40, 2048, [17, 40], torch.bfloat16, torch.int32),
                                                    (1, 33, 512, [20], torch.bfloat16, torch.int64), (3, 21, 1024, [21, 0, 5], torch.float16, torch.int64),
                                                    (5, 16, 7168, [0, 16, 3, 99, 1], torch.float16, torch.int32),
                                                    (3, 9, 36, [9, 0, 4], torch.bfloat16, torch.int64)])
def test_mask_quant_pack_matches_oracle(G, M, n, counts, dtype, mdt):
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    x = _x(G * M, n, dtype, seed=G).reshape(G, M, 2 * n)
    mask = torch.tensor(counts, dtype=mdt)
    packed_ref, written = R.fused_silu_mul_dq_mask_quant(x, mask)
    stride = R.silu_mul_pack_stride(2 * n)
    out = torch.full((G, M, stride), 3.0, dtype=dtype, device=DEV)   # byte pattern that must survive where nothing is written
    before = out.cpu().view(torch.uint8).reshape(G, M, stride * 2).clone()
    op.fused_silu_mul_dq_mask_quant(out, x.to(DEV), mask.to(DEV))
    got = out.cpu().view(torch.uint8).reshape(G, M, stride * 2)
    w = written
    if bool(w.any()):
        C.assert_codes(got[w][:, :n].contiguous().view(torch.int8), packed_ref[w][:, :n].contiguous().view(torch.int8))
        C.assert_close(got[w][:, n:n + 4].contiguous().view(torch.float32).reshape(-1),
                       packed_ref[w][:, n:n + 4].contiguous().view(torch.float32).reshape(-1), rel=1e-5, abs_=1e-9)
        assert torch.equal(got[w][:, n + 4:], before[w][:, n + 4:])          # padding of a written row stays as it was
    assert torch.equal(got[~w], before[~w])                                # rows beyond the count are untouched


@pytest.mark.gpu
def test_rejects_wrong_dtypes():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    x = _x(4, 64, torch.bfloat16).to(DEV)
    with pytest.raises(RuntimeError):
        op.fused_silu_mul_dq_reorder_quant(torch.empty(4, 64, dtype=torch.int8, device=DEV), torch.empty(4, device=DEV), x,
                                           torch.zeros(4, dtype=torch.float32, device=DEV), torch.empty(0), 0, 1)
    with pytest.raises(RuntimeError):
        op.fused_silu_mul_dq_mask_quant(torch.empty(1, 4, 256, dtype=torch.float16, device=DEV), x.reshape(1, 4, 128),
                                        torch.tensor([4], device=DEV))
