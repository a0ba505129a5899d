"""torch.ops._moe_C.grouped_topk (vLLM's grouped router with a score-correction bias): the oracle against the golden
vectors of the reference's biased_grouped_topk (the same routing rule), and the CUDA kernel against the oracle (ids
exact up to the float64-margin rule for near-ties, values to 1e-5 relative)."""
import pytest
import torch

from oracle import compare as C
from oracle import ref_ops as R
from tests.golden_io import records


def test_oracle_matches_biased_grouped_topk(golden):
    recs = [(k, r) for k, r in records(golden, "ref:unit_test/test_fused_moe_gate_deepseek.py:biased_grouped_topk")
            if r["gating"].dtype == torch.float32]
    assert len(recs) == 2
    for key, r in recs:
        w, ids = R.grouped_topk(r["gating"], 8, 4, 8, True, float(r["scaling"]), r["bias"], 1)
        C.assert_equal(torch.sort(ids, dim=1).values, torch.sort(r["ids"], dim=1).values, key)
        assert torch.allclose(torch.sort(w, dim=1).values, torch.sort(r["weights"], dim=1).values, rtol=1e-3, atol=1e-3), key


def test_oracle_scoring_none_and_the_uniform_fallback():
    g = torch.Generator().manual_seed(9)
    x = torch.randn(12, 64, generator=g)
    bias = torch.randn(64, generator=g) * 0.1
    s = 0.5 * torch.tanh(0.5 * x) + 0.5
    w1, i1 = R.grouped_topk(x, 4, 2, 6, True, 2.0, bias, 1)
    w0, i0 = R.grouped_topk(s, 4, 2, 6, True, 2.0, bias, 0)        # scores already activated
    assert torch.equal(i0, i1) and torch.allclose(w0, w1)
    assert torch.allclose(w1.sum(-1), torch.full((12,), 2.0), atol=1e-5)
    w2, _ = R.grouped_topk(x, 4, 2, 6, False, 2.0, bias, 1)
    assert torch.allclose(w2, torch.gather(s, 1, i1.long()) * 2.0, rtol=1e-6)
    # three of four groups are -inf everywhere: the second best group score is -inf -> ids 0..k-1, values 1/k
    y = x.clone()
    y[3, 16:] = -float("inf")
    w3, i3 = R.grouped_topk(y, 4, 2, 6, True, 2.0, bias, 0)
    assert i3[3].tolist() == list(range(6)) and torch.allclose(w3[3], torch.full((6,), 1.0 / 6))
    assert torch.equal(i3[:3], R.grouped_topk(x, 4, 2, 6, True, 2.0, bias, 0)[1][:3])


CASES = [(300, 256, 8, 4, 8, 2.5, 1, torch.float32, torch.float32), (64, 256, 8, 4, 8, 1.0, 0, torch.float32, torch.float32),
         (100, 128, 4, 2, 6, 1.5, 1, torch.float32, torch.float32), (50, 384, 1, 1, 8, 1.0, 1, torch.float32, torch.float32),
         (200, 256, 8, 4, 8, 2.5, 1, torch.bfloat16, torch.float32), (200, 256, 8, 4, 8, 2.5, 1, torch.float16, torch.float16),
         (8192, 256, 8, 4, 8, 2.5, 1, torch.float32, torch.float32)]


@pytest.mark.gpu
@pytest.mark.parametrize("n,E,G,TG,k,scaling,scoring,dtype,bdtype", CASES)
@pytest.mark.parametrize("renorm", [True, False])
def test_kernel_matches_oracle(n, E, G, TG, k, scaling, scoring, dtype, bdtype, renorm):
    import mcoplib_b200  # noqa: F401
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    g = torch.Generator().manual_seed(n + E + k)
    x = torch.randn(n, E, generator=g).to(dtype)
    bias = (torch.randn(E, generator=g) * 0.01).to(bdtype)
    w_ref, ids_ref = R.grouped_topk(x, G, TG, k, renorm, scaling, bias, scoring)
    if n % 2:
        w, ids = op.grouped_topk(x.to(DEV), G, TG, k, renorm, scaling, bias.to(DEV), scoring)
    else:
        w, ids = getattr(torch.ops, op.torch_moe_namespace).grouped_topk(x.to(DEV), G, TG, k, renorm, scaling, bias.to(DEV), scoring)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32 and w.shape == (n, k)
    w, ids = w.cpu(), ids.cpu()
    same = (ids == ids_ref).all(-1)
    if dtype == torch.float32 and scoring == 1:
        gap_g, gap_e = R.gate_margins(x, bias, k, G, TG)
        excused = C.assert_ids_with_margin(ids, ids_ref, torch.cat([gap_g.unsqueeze(1), gap_e], 1), torch.ones(n), "grouped_topk ids")
        assert excused <= 2
    else:
        # 16-bit scores: CUDA tanhf and the CPU tanh differ by an fp32 ulp or two before the rounding to 16 bits, and a score
        # that lands on the other side of a rounding boundary reorders the many exact ties of 16-bit scores
        assert int((~same).sum()) <= max(3, n // 20)
    C.assert_close(w[same], w_ref[same], "grouped_topk values", rel=1e-5 if dtype == torch.float32 else 1e-2, abs_=1e-6)


@pytest.mark.gpu
def test_uniform_fallback_and_non_finite_logits():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    g = torch.Generator().manual_seed(2)
    x = torch.randn(16, 256, generator=g)
    bias = torch.zeros(256)
    x[5, 32:] = -float("inf")          # one finite group only: the fourth best group score is -inf
    x[7, 3] = float("nan")             # a non-finite logit never wins a slot
    x[7, 40] = float("inf")
    w_ref, ids_ref = R.grouped_topk(x, 8, 4, 8, True, 1.0, bias, 0)
    w, ids = op.grouped_topk(x.to(DEV), 8, 4, 8, True, 1.0, bias.to(DEV), 0)
    assert ids.cpu()[5].tolist() == list(range(8)) and torch.allclose(w.cpu()[5], torch.full((8,), 0.125))
    keep = torch.ones(16, dtype=torch.bool); keep[7] = False
    C.assert_equal(ids.cpu()[keep], ids_ref[keep]); C.assert_close(w.cpu()[keep], w_ref[keep], rel=1e-5, abs_=1e-7)
    assert 3 not in ids.cpu()[7].tolist() and 40 not in ids.cpu()[7].tolist()


@pytest.mark.gpu
def test_rejects_what_the_reference_rejects():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    x = torch.randn(4, 256, device=DEV); b = torch.zeros(256, device=DEV)
    with pytest.raises(RuntimeError, match="divisible"):
        op.grouped_topk(x, 7, 2, 8, True, 1.0, b, 1)
    with pytest.raises(RuntimeError, match="scoring_func"):
        op.grouped_topk(x, 8, 4, 8, True, 1.0, b, 2)
    with pytest.raises(RuntimeError, match="2D"):
        op.grouped_topk(x.reshape(2, 2, 256), 8, 4, 8, True, 1.0, b, 1)
