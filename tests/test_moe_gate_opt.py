"""fused_moe_gate_opt (sglang-flavoured grouped sigmoid gate with an optional fused shared expert): the oracle against
the golden vectors made by the reference test's own biased_grouped_topk, and the CUDA kernel against the oracle
(ids exact up to the float64-margin rule for near-ties, weights to 1e-6 relative)."""
import pytest
import torch

from oracle import compare as C
from oracle import ref_ops as R
from tests.golden_io import records


def _tie_rows(gating, bias, G, TG, routed):
    """Rows whose result depends on how exact ties are broken (frequent for bf16 scores): torch.topk leaves the
    order of equal values open, the kernel contract sends ties to the lower index."""
    _, biased, _, ST = R._gate_scores(gating, bias)
    n, E = biased.shape
    tie = torch.zeros(n, dtype=torch.bool)
    masked = biased
    if G > 1:
        grp = biased.reshape(n, G, E // G)
        top2 = torch.sort(grp, dim=-1, descending=True).values[..., :2]
        gs = R.rt(top2[..., 0] + top2[..., 1], ST)
        gss = torch.sort(gs, dim=-1, descending=True).values
        tie |= gss[:, TG - 1] == gss[:, TG]
        _, gidx = R.stable_topk(gs, TG)
        gmask = torch.zeros(n, G, dtype=torch.bool).scatter_(1, gidx, True)
        emask = gmask.unsqueeze(-1).expand(n, G, E // G).reshape(n, E)
        masked = torch.where(emask, biased, torch.full_like(biased, -1e30))
    srt = torch.sort(masked, dim=-1, descending=True).values
    return tie | (srt[:, routed - 1] == srt[:, routed])


def test_oracle_matches_biased_grouped_topk(golden):
    recs = records(golden, "ref:unit_test/test_fused_moe_gate_opt.py:biased_grouped_topk")
    assert len(recs) == 6
    for key, r in recs:
        G, TG, k, shared = int(r["groups"]), int(r["topk_group"]), int(r["topk"]), int(r["shared"])
        w, ids = R.fused_moe_gate_opt(r["gating"], r["bias"], k, True, G, TG, shared, float(r["scaling"]))
        keep = ~_tie_rows(r["gating"], r["bias"], G, TG, k - shared)
        if r["gating"].dtype == torch.float32:
            assert bool(keep.all()), key
        assert int(keep.sum()) * 2 >= keep.numel(), key
        # the reference test compares row-sorted ids exactly and row-sorted weights by cosine similarity / 1e-3
        # (unit_test/test_fused_moe_gate_opt.py:167-172, 186-190)
        C.assert_equal(torch.sort(ids, dim=1).values[keep], torch.sort(r["ids"], dim=1).values[keep], key)
        tol = 1e-3 if r["gating"].dtype == torch.float32 else 1e-2   # bf16 weights: one bf16 ulp
        assert torch.allclose(torch.sort(w, dim=1).values[keep], torch.sort(r["weights"], dim=1).values[keep], rtol=tol, atol=tol), key
        if shared:
            assert bool((ids[:, -1] == r["gating"].shape[1]).all())
            assert torch.allclose(w[:, -1], torch.full((w.shape[0],), 1.0 / float(r["scaling"])), rtol=1e-2), key


def test_oracle_without_renormalisation_returns_scores_and_a_zero_shared_weight():
    g = torch.Generator().manual_seed(1)
    gating = torch.randn(8, 320, generator=g)
    bias = torch.randn(320, generator=g) * 0.01
    w, ids = R.fused_moe_gate_opt(gating, bias, 9, False, 1, 1, 1, 2.0)
    score = torch.sigmoid(gating)
    assert torch.allclose(w[:, :8], torch.gather(score, 1, ids[:, :8].long()), rtol=1e-6)
    assert float(w[:, 8].abs().max()) == 0.0 and bool((ids[:, 8] == 320).all())


CASES = [(64, 256, 8, 4, 8, 0, 1.0, torch.float32), (64, 256, 8, 4, 9, 1, 2.5, torch.float32), (33, 160, 1, 1, 8, 0, 1.0, torch.float32),
         (33, 160, 1, 1, 9, 1, 3.0, torch.bfloat16), (17, 320, 1, 1, 8, 0, 1.0, torch.float16), (17, 384, 1, 1, 9, 1, 1.0, torch.bfloat16),
         (2000, 448, 1, 1, 8, 0, 1.0, torch.float32), (8192, 256, 8, 4, 8, 0, 2.5, torch.bfloat16)]


@pytest.mark.gpu
@pytest.mark.parametrize("n,E,G,TG,k,shared,scaling,dtype", CASES)
@pytest.mark.parametrize("renorm", [True, False])
def test_kernel_matches_oracle(n, E, G, TG, k, shared, scaling, dtype, renorm):
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    g = torch.Generator().manual_seed(n + E + k)
    gating = torch.randn(n, E, generator=g).to(dtype)
    bias = (torch.randn(E, generator=g) * 0.01).to(dtype)
    w_ref, ids_ref = R.fused_moe_gate_opt(gating, bias, k, renorm, G, TG, shared, scaling)
    w = torch.full((n, k), -1.0, device=DEV)
    ids = torch.full((n, k), -1, dtype=torch.int32, device=DEV)
    rc = op.fused_moe_gate_opt(gating.to(DEV), bias.to(DEV), w, ids, k, renorm, G, TG, shared if shared else None, scaling)
    assert rc == 0
    routed = k - shared
    w, ids = w.cpu(), ids.cpu()
    same = (ids == ids_ref).all(-1)
    if dtype == torch.float32:
        gap_g, gap_e = R.gate_margins(gating, bias, routed, G, TG)
        excused = C.assert_ids_with_margin(ids[:, :routed], ids_ref[:, :routed], torch.cat([gap_g.unsqueeze(1), gap_e], 1),
                                           torch.ones(n), "gate_opt ids")
        assert excused <= 2
        C.assert_close(w[same], w_ref[same], "gate_opt weights", rel=1e-5, abs_=1e-7)
    else:
        # the CUDA and CPU sigmoid differ by an fp32 ulp before the rounding to 16 bits: a row whose 16-bit score sits on a
        # rounding boundary may differ; such rows must stay rare, all others agree exactly in ids (ties to the lower index)
        assert int((~same).sum()) <= max(3, n // 200)
        C.assert_close(w[same], w_ref[same], "gate_opt weights", rel=1e-2, abs_=1e-3)
    if shared:
        assert bool((ids[:, -1] == E).all())
    if renorm:
        assert torch.allclose(w[:, :routed].sum(-1), torch.ones(n), atol=2e-2)


@pytest.mark.gpu
def test_rejects_what_the_reference_rejects():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    gating = torch.randn(4, 256, device=DEV); bias = torch.zeros(256, device=DEV)
    w8 = torch.empty(4, 8, device=DEV); i8 = torch.empty(4, 8, dtype=torch.int32, device=DEV)
    w9 = torch.empty(4, 9, device=DEV); i9 = torch.empty(4, 9, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="Expected topk = 8"):
        op.fused_moe_gate_opt(gating, bias, torch.empty(4, 6, device=DEV), torch.empty(4, 6, dtype=torch.int32, device=DEV), 6, True, 8, 4)
    with pytest.raises(RuntimeError, match="Expected topk == 8"):
        op.fused_moe_gate_opt(gating, bias, w9, i9, 9, True, 8, 4)
    with pytest.raises(RuntimeError, match="Expected topk >= 9"):
        op.fused_moe_gate_opt(gating, bias, w8, i8, 8, True, 8, 4, 1, 2.5)
    with pytest.raises(RuntimeError, match="Invalid arguments"):
        op.fused_moe_gate_opt(gating, bias, w8, i8, 8, True, 4, 2)
    with pytest.raises(RuntimeError, match="rand"):
        op.fused_moe_gate_opt(gating, bias, w9, i9, 9, True, 8, 4, 2, 2.5)
