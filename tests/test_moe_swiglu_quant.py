"""moe_swiglu_dynamic_quantize (the step after the expert up-projection): the oracle against the golden vector made
by the reference's own torch reference, and the CUDA kernel against the oracle (codes +-1 LSB on <= 0.01 %: the CPU
exp and the CUDA expf differ in the last ulp; scales 1e-5 relative)."""
import pytest
import torch

from mcoplib_b200 import workloads as W
from oracle import compare as C
from oracle import ref_ops as R
from tests.golden_io import records


def test_oracle_matches_reference_torch_function(golden):
    (key, r), = records(golden, "ref:unit_test/test_moe_swiglu_dq.py:moe_swiglu_dynamic_quant_run")
    q, s = R.moe_swiglu_dynamic_quantize(r["x"], r["smooth"], r["starts"], r["counts"], 4)
    assert C.code_stats(q, r["codes"])["max_abs"] <= 1, key      # the reference test's tolerance (atol 1)
    assert C.code_stats(q, r["codes"])["frac_diff"] < 1e-3, key
    assert torch.allclose(s, r["scales"], rtol=1e-5), key


def _case(rows_per_expert, H, seed=0):
    counts = torch.tensor(rows_per_expert, dtype=torch.int32)
    starts = (torch.cumsum(counts, 0) - counts).to(torch.int32)
    rows = int(counts.sum())
    x = W.per_token("randn", 70, 0, max(rows, 1), 2 * H, torch.bfloat16, seed=seed)[:rows]
    smooth = 0.5 + torch.rand(len(rows_per_expert), H, generator=torch.Generator().manual_seed(seed))
    return x, smooth, starts, counts


@pytest.mark.gpu
@pytest.mark.parametrize("rows_per_expert,H", [([5, 0, 9, 6], 256), ([300, 200, 0, 17, 1], 2048), ([64] * 8, 7168),
                                                ([3, 4], 100), ([10, 10], 16384), ([0, 0, 7], 520), ([7, 3, 0, 50], 1024), ([1, 2, 2], 2048)])
def test_kernel_matches_oracle(rows_per_expert, H):
    from mcoplib_b200 import op
    from tests.gpu_util import DEV, Canary
    x, smooth, starts, counts = _case(rows_per_expert, H)
    E, rows = len(rows_per_expert), x.shape[0]
    x[1] = 0                                            # an all-zero row: codes 0, scale 0
    q_ref, s_ref = R.moe_swiglu_dynamic_quantize(x, smooth, starts, counts, E)
    y = Canary((rows, H), torch.int8); sc = Canary((rows,), torch.float32)
    op.moe_swiglu_dynamic_quantize(x.to(DEV), smooth.to(DEV), starts.to(DEV), counts.to(DEV), y.t, sc.t, E)
    torch.cuda.synchronize()
    y.check(); sc.check()
    C.assert_codes(y.t, q_ref); C.assert_close(sc.t, s_ref, rel=1e-5, abs_=1e-9)
    assert int(y.t[1].abs().max()) == 0 and float(sc.t[1]) == 0.0


@pytest.mark.gpu
def test_rows_outside_every_expert_are_left_alone():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    x, smooth, _, _ = _case([20, 20], 512)
    starts = torch.tensor([0, 25], dtype=torch.int32); counts = torch.tensor([10, 15], dtype=torch.int32)   # rows 10..24 unowned
    q_ref, s_ref = R.moe_swiglu_dynamic_quantize(x, smooth, starts, counts, 2)
    y = torch.full((40, 512), 7, dtype=torch.int8, device=DEV); sc = torch.full((40,), -1.0, device=DEV)
    op.moe_swiglu_dynamic_quantize(x.to(DEV), smooth.to(DEV), starts.to(DEV), counts.to(DEV), y, sc, 2)
    own = torch.zeros(40, dtype=torch.bool); own[:10] = True; own[25:] = True
    C.assert_codes(y.cpu()[own], q_ref[own]); C.assert_close(sc.cpu()[own], s_ref[own], rel=1e-5, abs_=1e-9)
    assert bool((y.cpu()[~own] == 7).all()) and bool((sc.cpu()[~own] == -1.0).all())
