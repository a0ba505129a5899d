"""Comparison rules shared by the parity tests.  TEST INFRASTRUCTURE ONLY (see ref_ops.py).

Tolerances (stated once here, used everywhere):
  * expert ids, group masks, permutations, counts, starts, gather indices: bit-exact.  An id
    mismatch is excused only if the float64 decision margin of that row is below `ULP_EXCUSE`
    fp32 ulps (CPU exp and CUDA expf are not bit-identical); excused rows are counted and reported.
  * int8 codes: |a-b| <= 1 everywhere and a != b on at most 0.01 % of the elements.
  * fp32 scales and bf16 outputs: |a-b| <= 1e-3 + 1e-2 * |b|.
"""
from __future__ import annotations

import math

import torch

CODE_MISMATCH_FRACTION = 1e-4
REL_TOL = 1e-2
ABS_TOL = 1e-3
ULP_EXCUSE = 8.0


def code_stats(a: torch.Tensor, b: torch.Tensor):
    d = (a.to(torch.int16) - b.to(torch.int16)).abs()
    n = d.numel()
    return {"n": n, "max_abs": int(d.max()) if n else 0, "n_diff": int((d != 0).sum()),
            "frac_diff": (float((d != 0).sum()) / n) if n else 0.0}


def assert_codes(a: torch.Tensor, b: torch.Tensor, what: str = "codes", frac: float = CODE_MISMATCH_FRACTION):
    """+-1 LSB on at most `frac` of the elements (at least one element is always allowed so that the
    rule stays meaningful for tensors smaller than 1/frac)."""
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    st = code_stats(a.cpu(), b.cpu())
    assert st["max_abs"] <= 1, f"{what}: max |diff| {st['max_abs']} > 1 LSB ({st})"
    allowed = max(1, math.floor(frac * st["n"]))
    assert st["n_diff"] <= allowed, f"{what}: {st['n_diff']} of {st['n']} codes differ (> {allowed})"
    return st


def assert_close(a: torch.Tensor, b: torch.Tensor, what: str = "values", rel: float = REL_TOL, abs_: float = ABS_TOL):
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    af, bf = a.detach().cpu().float(), b.detach().cpu().float()
    err = (af - bf).abs()
    lim = abs_ + rel * bf.abs()
    bad = err > lim
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} of {bad.numel()} outside tol; "
                                 f"max err {float(err.max()):.4g} at ref {float(bf.flatten()[err.argmax()]):.4g}")
    return float(err.max()) if err.numel() else 0.0


def assert_equal(a: torch.Tensor, b: torch.Tensor, what: str = "ints"):
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    a, b = a.cpu(), b.cpu()
    if not torch.equal(a, b):
        bad = torch.nonzero((a != b).reshape(-1))[:5].reshape(-1).tolist()
        raise AssertionError(f"{what}: {int((a != b).sum())} of {a.numel()} differ, first at flat {bad}: "
                             f"{a.reshape(-1)[bad].tolist()} vs {b.reshape(-1)[bad].tolist()}")


def ulp32(v: torch.Tensor) -> torch.Tensor:
    """Size of one fp32 ulp at |v| (float64 tensor in, float64 out)."""
    f = v.abs().float().clamp_min(torch.finfo(torch.float32).tiny)
    return (torch.nextafter(f, torch.full_like(f, float("inf"))) - f).double()


def assert_ids_with_margin(ids: torch.Tensor, ref_ids: torch.Tensor, margins: torch.Tensor,
                           scale_ref: torch.Tensor, what: str = "ids"):
    """ids must equal ref_ids row by row.  A differing row is excused only if the smallest float64
    decision margin of that row (`margins` [rows, m]) is below ULP_EXCUSE fp32 ulps of the score
    magnitude `scale_ref` [rows].  Returns the number of excused rows."""
    ids, ref_ids = ids.cpu(), ref_ids.cpu()
    assert ids.shape == ref_ids.shape
    bad_rows = torch.nonzero((ids != ref_ids).any(dim=-1)).reshape(-1)
    if bad_rows.numel() == 0:
        return 0
    m = margins.reshape(margins.shape[0], -1).min(dim=1).values[bad_rows]
    lim = ULP_EXCUSE * ulp32(scale_ref.double()[bad_rows])
    unexcused = bad_rows[m > lim]
    assert unexcused.numel() == 0, (f"{what}: {unexcused.numel()} rows differ with a decision margin above "
                                    f"{ULP_EXCUSE} ulp, e.g. row {int(unexcused[0])}: {ids[unexcused[0]].tolist()} vs "
                                    f"{ref_ids[unexcused[0]].tolist()}")
    return int(bad_rows.numel())
