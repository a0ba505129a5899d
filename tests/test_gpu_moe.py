"""GPU parity of part 3 (routers, scatter with per-row int8 quant, gather) against the CPU oracle and the
golden vectors, through the operator shims over the C ABI.

Expert ids, group masks, permutations (row2tok / tok2row), counts, starts and gather results are compared
bit-exactly.  An id mismatch is excused only where the float64 decision margin is within a few fp32 ulps
(CPU exp vs CUDA expf); excused rows are counted and must stay a vanishing fraction."""
import pytest
import torch

from mcoplib_b200 import workloads as W
from oracle import compare as C
from oracle import ref_ops as R
from tests.golden_io import records
from tests.gpu_util import DEV, Canary, bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def op():
    from mcoplib_b200 import op as _op
    return _op


# ------------------------------------------------------------------------------------------ routers
def _softmax(op, logits, k):
    T = logits.shape[0]
    w = Canary((T, k), torch.float32); i = Canary((T, k), torch.int32)
    op.moe_softmax_topk(w.t, i.t, logits.to(DEV), False)
    torch.cuda.synchronize()
    w.check("weights"); i.check("ids")
    return w.t.cpu(), i.t.cpu()


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (32768, 8, 2), (777, 8, 1), (100, 4, 2), (100, 7, 3), (513, 16, 2), (300, 32, 4),
                                   (1000, 64, 6), (333, 60, 4), (257, 128, 8), (2000, 256, 8), (100, 160, 8), (64, 384, 8),
                                   (50, 512, 8), (40, 1024, 8), (20, 1000, 32)])
def test_softmax_topk_matches_oracle(op, T, E, k):
    x = W.router_inputs(T, E)["logits"]
    w_ref, ids_ref = R.moe_softmax_topk(x, k)
    w, ids = _softmax(op, x, k)
    excused = C.assert_ids_with_margin(ids, ids_ref, R.softmax_topk_margin(x, k), x.abs().amax(-1), "softmax ids")
    assert excused <= max(1, T // 10000)
    same = (ids == ids_ref).all(-1)
    C.assert_close(w[same], w_ref[same], "softmax weights", rel=1e-4, abs_=1e-6)
    assert torch.allclose(w.sum(-1), torch.ones(T), atol=1e-5)      # always renormalised
    assert bool((w[:, :-1] >= w[:, 1:]).all())                       # descending order


def test_softmax_topk_ties_go_to_the_lowest_index(op):
    x = torch.zeros(64, 8)
    x[1, 3] = x[1, 6] = 2.0
    x[2] = torch.tensor([1., 5., 5., 5., 0., 0., 5., 1.])
    w, ids = _softmax(op, x, 2)
    assert ids[0].tolist() == [0, 1] and ids[1].tolist() == [3, 6] and ids[2].tolist() == [1, 2]
    w_ref, ids_ref = R.moe_softmax_topk(x, 2)
    C.assert_equal(ids, ids_ref); C.assert_close(w, w_ref)
    # rows of a warp must not alias when several rows share a warp (E <= 32)
    x = W.router_inputs(96, 8)["logits"]
    C.assert_equal(_softmax(op, x, 2)[1], R.moe_softmax_topk(x, 2)[1])


def test_softmax_topk_against_golden(op, golden):
    for key, g in records(golden, "formula:benchmark/runners/mcoplib_mxbenchmark_topk_softmax_runners.py:38-49"):
        w, ids = _softmax(op, g["gating"], g["k"])
        C.assert_equal(ids, g["ids"], key)
        assert torch.allclose(w, g["weights"], rtol=1e-4, atol=1e-6), key


def _gate(op, logits, bias, topk, G, tg, scaling, renorm=True):
    T = logits.shape[0]
    w = Canary((T, topk), torch.float32); i = Canary((T, topk), torch.int32); gm = Canary((T,), torch.int32)
    rc = op.fused_moe_gate_deepseek(logits.to(DEV), bias.to(DEV), w.t, i.t, topk, renorm, G, tg, None, scaling, 0, gm.t)
    torch.cuda.synchronize()
    assert rc == 0
    w.check(); i.check(); gm.check()
    return w.t.cpu(), i.t.cpu(), gm.t.cpu()


def test_config3_gate(op):
    """Benchmark configuration 3: 8192 tokens, 256 experts, 8 groups, top-4 groups, top-8, scaling 2.5."""
    d = W.router_inputs(8192, 256)
    w_ref, ids_ref, gm_ref = R.fused_moe_gate_deepseek(d["logits"], d["bias"], 8, True, 8, 4, 2.5)
    w, ids, gm = _gate(op, d["logits"], d["bias"], 8, 8, 4, 2.5)
    gap_g, gap_e = R.gate_margins(d["logits"], d["bias"], 8, 8, 4)
    excused = C.assert_ids_with_margin(ids, ids_ref, torch.cat([gap_g.unsqueeze(1), gap_e], 1), torch.ones(8192), "gate ids")
    assert excused <= 2
    same = (ids == ids_ref).all(-1)
    C.assert_equal(gm[same], gm_ref[same], "group mask"); C.assert_close(w[same], w_ref[same], "gate weights", rel=1e-4, abs_=1e-6)
    assert torch.allclose(w.sum(-1), torch.full((8192,), 2.5), atol=1e-4)
    assert bool(((gm.unsqueeze(1) >> torch.arange(8).unsqueeze(0)) & 1).sum(1).eq(4).all())


@pytest.mark.parametrize("E,G,tg,topk", [(256, 8, 4, 8), (256, 8, 8, 8), (256, 1, 1, 8), (320, 1, 1, 8), (384, 1, 1, 8), (448, 1, 1, 8),
                                          (128, 4, 2, 4), (64, 8, 3, 6), (512, 16, 4, 8), (256, 8, 4, 5)])
@pytest.mark.parametrize("renorm", [True, False])
def test_gate_shapes(op, E, G, tg, topk, renorm):
    d = W.router_inputs(300, E)
    w_ref, ids_ref, gm_ref = R.fused_moe_gate_deepseek(d["logits"], d["bias"], topk, renorm, G, tg, 1.5)
    w, ids, gm = _gate(op, d["logits"], d["bias"], topk, G, tg, 1.5, renorm)
    gap_g, gap_e = R.gate_margins(d["logits"], d["bias"], topk, G, tg)
    excused = C.assert_ids_with_margin(ids, ids_ref, torch.cat([gap_g.unsqueeze(1), gap_e], 1), torch.ones(300), "gate ids")
    assert excused <= 1
    same = (ids == ids_ref).all(-1)
    C.assert_close(w[same], w_ref[same], rel=1e-4, abs_=1e-6); C.assert_equal(gm[same], gm_ref[same])


def test_gate_logits_that_start_off_a_16_byte_boundary(op):
    """A contiguous fp32 logits view whose first element sits 4 bytes into its storage: the 16-byte loads of the fast
    path do not apply, the gate must take element loads and produce the same result."""
    d = W.router_inputs(300, 256)
    w_ref, ids_ref, gm_ref = R.fused_moe_gate_deepseek(d["logits"], d["bias"], 8, True, 8, 4, 2.5)
    flat = torch.zeros(300 * 256 + 1, device=DEV)
    view = flat[1:].view(300, 256)
    view.copy_(d["logits"])
    assert view.is_contiguous() and view.data_ptr() % 16 == 4
    w = torch.empty(300, 8, device=DEV); i = torch.empty(300, 8, dtype=torch.int32, device=DEV)
    op.fused_moe_gate_deepseek(view, d["bias"].to(DEV), w, i, 8, True, 8, 4, None, 2.5, 0)
    w0, i0, _ = _gate(op, d["logits"], d["bias"], 8, 8, 4, 2.5)
    C.assert_equal(i.cpu(), i0); C.assert_equal(bits(w.cpu()), bits(w0))


@pytest.mark.parametrize("dtype,bias_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16),
                                              (torch.bfloat16, torch.float32), (torch.float16, torch.float32)])
def test_gate_half_precision_logits(op, dtype, bias_dtype):
    """Reduced-precision scores tie often; ties must go to the lower index exactly as in the oracle.  The CUDA and
    CPU sigmoid differ by an fp32 ulp before the rounding to 16 bits, so a row whose 16-bit score sits on a rounding
    boundary may differ: such rows must stay rare."""
    g = torch.Generator().manual_seed(4)
    logits = torch.rand(256, 256, generator=g).to(dtype); bias = torch.rand(256, generator=g).to(bias_dtype)
    w_ref, ids_ref, gm_ref = R.fused_moe_gate_deepseek(logits, bias, 8, True, 8, 4, 1.0)
    w, ids, gm = _gate(op, logits, bias, 8, 8, 4, 1.0)
    same = (ids == ids_ref).all(-1)
    assert int((~same).sum()) <= 3
    C.assert_equal(gm[same], gm_ref[same]); C.assert_close(w[same], w_ref[same], rel=1e-2, abs_=1e-3)


@pytest.mark.parametrize("E,G,tg", [(256, 8, 4), (384, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shared,renorm", [(0, True), (0, False), (1, True), (1, False)])
def test_gate_sglang_form_with_fused_shared_expert(op, E, G, tg, dtype, shared, renorm):
    """moegate_type 1 of fused_moe_gate_deepseek: unscaled weights, optional fused shared expert in the last slot."""
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(300, E, generator=g).to(dtype)
    bias = (0.01 * torch.randn(E, generator=g)).to(dtype)
    topk = 8 + shared
    w_ref, ids_ref = R.fused_moe_gate_deepseek_sglang(logits, bias, topk, renorm, G, tg, 2.5, shared)
    w = torch.empty(300, topk, device=DEV); i = torch.empty(300, topk, dtype=torch.int32, device=DEV)
    rc = op.fused_moe_gate_deepseek(logits.to(DEV), bias.to(DEV), w, i, topk, renorm, G, tg, shared, 2.5, 1)
    assert rc == 0
    w, i = w.cpu(), i.cpu()
    same = (i == ids_ref).all(-1)
    assert int((~same).sum()) <= (0 if dtype == torch.float32 else 3)   # 16-bit scores tie on rounding boundaries
    if shared:
        assert bool((i[:, -1] == E).all())
    tol = dict(rel=1e-5, abs_=1e-7) if dtype == torch.float32 else dict(rel=1e-2, abs_=1e-3)
    C.assert_close(w[same], w_ref[same], "sglang-form weights", **tol)
    with pytest.raises(RuntimeError):   # shared experts exist only in the SGLANG form; two of them are not built
        op.fused_moe_gate_deepseek(logits.to(DEV), bias.to(DEV), w.to(DEV), i.to(DEV), 9, renorm, G, tg, 1, 2.5, 0)
    with pytest.raises(RuntimeError):
        op.fused_moe_gate_deepseek(logits.to(DEV), bias.to(DEV), w.to(DEV), i.to(DEV), 9, renorm, G, tg, 2, 2.5, 1)


def test_gate_against_golden(op, golden):
    """The reference test's own criterion: row-sorted ids equal, row-sorted weights within 1e-3."""
    for key, g in records(golden, "ref:unit_test/test_fused_moe_gate_deepseek.py:biased_grouped_topk"):
        if g["gating"].dtype != torch.float32:
            continue
        w, ids, _ = _gate(op, g["gating"], g["bias"], 8, 8, 4, g["scaling"])
        C.assert_equal(torch.sort(ids, dim=1).values, torch.sort(g["ids"], dim=1).values, key)
        assert torch.allclose(torch.sort(w, dim=1).values, torch.sort(g["weights"], dim=1).values, rtol=1e-3, atol=1e-3), key


def test_gate_rejects_unsupported_configurations(op):
    d = W.router_inputs(4, 250)
    with pytest.raises(RuntimeError):
        _gate(op, d["logits"], d["bias"], 8, 1, 1, 1.0)
    d = W.router_inputs(4, 256)
    with pytest.raises(RuntimeError):
        _gate(op, d["logits"], d["bias"], 8, 8, 0, 1.0)
    with pytest.raises(RuntimeError):
        op.fused_moe_gate_deepseek(d["logits"].to(DEV), d["bias"].to(DEV), torch.empty(4, 8, device=DEV),
                                   torch.empty(4, 8, dtype=torch.int32, device=DEV), 8, True, 8, 4, 1, 1.0, 0)


# ------------------------------------------------------------------------------------------ dispatch
def _scatter(op, hidden, ids, w, smooth, E, with_t2r=True):
    T, H = hidden.shape
    k = ids.shape[1]
    Rn = T * k
    rows = Canary((Rn, H), torch.int8, fill=0); sc = Canary((Rn,), torch.float32, fill=0)
    r2t = Canary((Rn,), torch.int32, fill=-1); cnt = Canary((E,), torch.int32); st = Canary((E,), torch.int32)
    t2r = Canary((T, k), torch.int32, fill=-7)
    op.moe_scatter_dynamic_quant(hidden.to(DEV), ids.to(DEV), w.to(DEV), smooth.to(DEV), rows.t, sc.t, r2t.t, cnt.t, st.t, E, 0, 0,
                                 t2r.t if with_t2r else None)
    torch.cuda.synchronize()
    for c in (rows, sc, r2t, cnt, st, t2r):
        c.check("scatter outputs")
    return rows.t, sc.t, r2t.t, cnt.t, st.t, t2r.t


def _check_scatter(op, T, H, E, k, ids=None, w=None, smooth=None, seed=0):
    if ids is None:
        w, ids = R.moe_softmax_topk(W.router_inputs(T, E, seed=seed)["logits"], k)
    d = W.dispatch_inputs(T, H, E, k, seed=seed)
    if smooth is None:
        smooth = 0.5 + torch.rand(E, H, generator=torch.Generator().manual_seed(seed))
    ref = R.moe_scatter_dynamic_quant(d["hidden"], ids, w, smooth, E)
    got = _scatter(op, d["hidden"], ids, w, smooth, E)
    rows_ref, sc_ref, r2t_ref, cnt_ref, st_ref, t2r_ref = ref
    rows, sc, r2t, cnt, st, t2r = got
    C.assert_equal(cnt, cnt_ref, "counts"); C.assert_equal(st, st_ref, "starts")
    C.assert_equal(r2t, r2t_ref, "row2tok"); C.assert_equal(t2r, t2r_ref, "tok2row")
    C.assert_close(sc, sc_ref, "row scales", rel=1e-5, abs_=1e-9); C.assert_codes(rows, rows_ref, "rows")
    return d, ids, w, ref, got


@pytest.mark.parametrize("T,H,E,k", [(1, 64, 8, 2), (511, 1024, 8, 2), (512, 1024, 8, 2), (513, 1024, 8, 2), (2000, 2048, 64, 6),
                                     (1500, 7168, 256, 8), (300, 520, 16, 4), (64, 100, 8, 2), (130, 16384, 8, 2), (40, 32768, 4, 1),
                                     (1030, 512, 200, 3), (1100, 4096, 8, 2), (600, 5120, 16, 4), (700, 6144, 8, 3), (1024, 8192, 8, 2),
                                     (33000, 256, 40, 3), (70000, 64, 256, 8)])  # the last two: more than 64 tiles (scan kernel)
def test_scatter_matches_oracle(op, T, H, E, k):
    _check_scatter(op, T, H, E, k)


def test_scatter_drops_foreign_experts_and_handles_empty_experts(op):
    T, H, E_total, E_local, k = 700, 1024, 16, 6, 4
    w, ids = R.moe_softmax_topk(W.router_inputs(T, E_total)["logits"], k)
    ids[ids == 2] = 9                                    # expert 2 receives nothing; ids >= E_local are dropped
    ids[5, 0] = -3                                       # negative ids are dropped too
    d = W.dispatch_inputs(T, H, E_local, k)
    smooth = 0.5 + torch.rand(E_local, H, generator=torch.Generator().manual_seed(1))
    ref = R.moe_scatter_dynamic_quant(d["hidden"], ids, w, smooth, E_local)
    rows, sc, r2t, cnt, st, t2r = _scatter(op, d["hidden"], ids, w, smooth, E_local)
    n = int(ref[3].sum())
    assert 0 < n < T * k and int(ref[3][2]) == 0
    C.assert_equal(cnt, ref[3]); C.assert_equal(st, ref[4]); C.assert_equal(t2r, ref[5])
    C.assert_equal(r2t[:n], ref[2][:n]); C.assert_codes(rows[:n], ref[0][:n]); C.assert_close(sc[:n], ref[1][:n], rel=1e-5, abs_=1e-9)
    assert bool((r2t[n:] == -1).all()) and int(rows[n:].abs().max()) == 0, "rows past the routed ones are left untouched"


def test_scatter_zero_rows_and_workspace_reuse(op):
    T, H, E, k = 600, 1024, 8, 2
    w, ids = R.moe_softmax_topk(W.router_inputs(T, E)["logits"], k)
    d = W.dispatch_inputs(T, H, E, k)
    d["hidden"][3] = 0                                   # all-zero token row: codes 0, scale 0
    smooth = torch.ones(E, H)
    ref = R.moe_scatter_dynamic_quant(d["hidden"], ids, w, smooth, E)
    for _ in range(3):                                   # repeated calls reuse the allocator's scratch block
        rows, sc, r2t, cnt, st, t2r = _scatter(op, d["hidden"], ids, w, smooth, E)
        C.assert_equal(r2t, ref[2]); C.assert_codes(rows, ref[0]); C.assert_close(sc, ref[1], rel=1e-5, abs_=1e-9)
    zr = t2r[3].long()
    assert float(sc[zr].abs().max()) == 0 and int(rows[zr].abs().max()) == 0


def test_scatter_row_quant_against_golden(op, golden):
    (key, g), = records(golden, "ref:unit_test/test_moe_swiglu_dq.py:smooth_per_token_dynamic_quant")
    n = g["hidden"].shape[0]
    rows, sc, r2t, cnt, st, _ = _scatter(op, g["hidden"], torch.zeros(n, 1, dtype=torch.int32), torch.ones(n, 1), g["smooth"].reshape(1, -1), 1)
    C.assert_equal(r2t, torch.arange(n, dtype=torch.int32), key)
    assert torch.allclose(sc.cpu(), g["scales"], rtol=1e-5), key
    assert C.code_stats(rows.cpu(), g["codes"])["max_abs"] <= 1, key


@pytest.mark.parametrize("T,H,E,k", [(700, 1024, 8, 2), (300, 7168, 256, 8), (33, 520, 16, 4), (200, 16384, 8, 2), (1, 64, 4, 1)])
def test_gather_matches_oracle_bit_for_bit(op, T, H, E, k):
    d, ids, w, ref, got = _check_scatter(op, T, H, E, k)
    r2t, st, t2r = got[2], got[4], got[5]
    y = d["y"]
    out0 = W.per_token("randn", 50, 0, T, H, torch.bfloat16)
    g_ref = R.moe_gather(y, ref[2], out0)
    for use in (False, True):
        o = Canary((T, H), torch.bfloat16); o.t.copy_(out0)
        op.moe_gather(y.to(DEV), r2t, o.t, t2r if use else None)
        torch.cuda.synchronize(); o.check("gather")
        C.assert_equal(bits(o.t), bits(g_ref), f"gather tok2row={use}")
    for acc in (False, True):
        gw_ref = R.moe_gather_weighted(y, ref[2], ids, w, ref[4], out0, acc)
        for use in (False, True):
            o = out0.clone().to(DEV)
            op.moe_gather_weighted(y.to(DEV), r2t, ids.to(DEV), w.to(DEV), st, o, acc, t2r if use else None)
            C.assert_equal(bits(o), bits(gw_ref), f"weighted gather accumulate={acc} tok2row={use}")
    # the fixed-order fp32 sum stays within bf16 rounding of one legal order of the reference's bf16 atomics
    seq = R.moe_gather_bf16_sequential(y[:min(len(y), 400)], ref[2][:min(len(y), 400)], out0) if T <= 300 else None
    if seq is not None and T * k <= 400:
        assert float((g_ref.float() - seq.float()).abs().max()) <= 0.02 * float(seq.float().abs().max()) + 1e-3


@pytest.mark.parametrize("T,H,E,k,local", [(1024, 7168, 8, 2, 8), (1500, 4096, 16, 4, 16), (4097, 4096, 64, 8, 64),
                                             (2049, 7168, 8, 1, 8), (9000, 4096, 8, 2, 6), (2500, 7168, 32, 8, 20)])
def test_gather_pipelined_with_tok2row_matches_oracle(op, T, H, E, k, local):
    """The pipelined gather (1024 tokens and more, rows of 2056 ... 16,384 elements) with the direct inverse map: every
    CTA walks its share in several chunks with a ragged last one and makes the next chunk's row lists while the current
    one streams.  `local` < E drops the rows of the experts beyond it (tok2row = -1 there), so tokens own 0 ... k rows.
    Plain and weighted, with and without accumulation, bit for bit against the oracle."""
    w, ids = R.moe_softmax_topk(W.router_inputs(T, E, seed=21)["logits"], k)
    r2t, cnt, st, t2r = R.moe_scatter_permutation(ids, local)
    Rn = T * k
    y = W.per_token("randn", 61, 0, Rn, H, torch.bfloat16)
    out0 = W.per_token("randn", 62, 0, T, H, torch.bfloat16)
    if local < E:
        assert int((t2r < 0).sum()) > 0
    o = Canary((T, H), torch.bfloat16); o.t.copy_(out0)
    op.moe_gather(y.to(DEV), r2t.to(DEV), o.t, t2r.to(DEV))
    torch.cuda.synchronize(); o.check("gather")
    C.assert_equal(bits(o.t), bits(R.moe_gather(y, r2t, out0)), "gather")
    for acc in (False, True):
        ref = R.moe_gather_weighted(y, r2t, ids, w, st, out0, acc)
        o = Canary((T, H), torch.bfloat16); o.t.copy_(out0)
        op.moe_gather_weighted(y.to(DEV), r2t.to(DEV), ids.to(DEV), w.to(DEV), st.to(DEV), o.t, acc, t2r.to(DEV))
        torch.cuda.synchronize(); o.check("weighted gather")
        C.assert_equal(bits(o.t), bits(ref), f"weighted gather accumulate={acc}")


def test_gather_fixed_order_against_legal_orders_of_the_reference_at_top8_hidden_7168(op):
    """The reference sums a token's rows with bf16 atomics in whatever order the hardware takes them; the build sums in
    fp32 in ascending row order and rounds once.  At the DeepSeek-V3 shape (8 rows per token, hidden 7168) the result
    must stay within the bf16 rounding noise of two legal orders of the reference (ascending and descending rows, a
    rounding after every add), and lie closer to the exact sum than either of them on average."""
    T, H, E, k = 256, 7168, 256, 8
    d = W.dispatch_inputs(T, H, E, k, seed=3)
    w, ids = R.moe_softmax_topk(W.router_inputs(T, E, seed=3)["logits"], k)
    r2t, cnt, st, t2r = R.moe_scatter_permutation(ids, E)
    y = d["y"]
    out0 = W.per_token("randn", 53, 0, T, H, torch.bfloat16)
    o = out0.clone().to(DEV)
    op.moe_gather(y.to(DEV), r2t.to(DEV), o, t2r.to(DEV))
    got = o.cpu().float()
    C.assert_equal(bits(o), bits(R.moe_gather(y, r2t, out0)), "fixed-order oracle")
    rows = torch.sort(t2r.long(), dim=1).values                     # ascending rows of every token
    exact = out0.double() + y[rows].double().sum(dim=1)
    def legal(order):
        acc = out0.clone()
        for j in order:
            acc = (acc.float() + y[rows[:, j]].float()).to(torch.bfloat16)
        return acc.float()
    asc, desc = legal(range(k)), legal(reversed(range(k)))
    scale = float(exact.abs().max())
    for name, ref in (("ascending", asc), ("descending", desc)):
        assert float((got - ref).abs().max()) <= 0.02 * scale + 1e-3, name
    err = lambda v: float((v.double() - exact).abs().mean())
    assert err(got) <= err(asc) and err(got) <= err(desc), "one rounding is closer to the exact sum than eight"


def test_gather_arbitrary_row_map(op):
    """The 3-argument operator accepts any row -> token map: unequal counts, a token owning more rows than the
    kernels' row tables hold (the slow scan), tokens with no rows, and entries outside [0, tokens) that are skipped."""
    T, H, Rn = 50, 1024, 400
    g = torch.Generator().manual_seed(8)
    r2t = torch.randint(0, T, (Rn,), generator=g).to(torch.int32)
    r2t[100:300] = 7                                     # token 7 owns ~200 rows
    r2t[r2t == 11] = 12                                  # token 11 owns none
    r2t[0] = -1; r2t[399] = T + 5                        # skipped
    y = W.per_token("randn", 51, 0, Rn, H, torch.bfloat16)
    out0 = W.per_token("randn", 52, 0, T, H, torch.bfloat16)
    ref = R.moe_gather(y, r2t, out0)
    o = out0.clone().to(DEV)
    op.moe_gather(y.to(DEV), r2t.to(DEV), o)
    C.assert_equal(bits(o), bits(ref))
    assert torch.equal(bits(o[11]), bits(out0[11]))


@pytest.mark.parametrize("T,H", [(4096, 4096), (300, 1024)])
def test_gather_skewed_map_without_tok2row(op, T, H):
    """The expert-parallel case of the 3-argument operator: three quarters of the routing rows were dropped, so the map holds
    about two rows per token on average while the tokens that kept theirs own eight (and a few own 12, 16 and 17: at, and
    one past, what the pipelined kernel's table holds; 40 and 70: around what the row-per-CTA kernels hold).  The inverse
    is a chain per token, exact whatever the spread; bit-exact against the oracle at both sizes (the pipelined kernel from
    1024 tokens, one CTA per token below)."""
    g = torch.Generator().manual_seed(9)
    owners = torch.randperm(T, generator=g)[: T // 4]
    r2t = owners.repeat_interleave(8)
    extra = torch.cat([owners[:1].repeat(4), owners[1:2].repeat(8), owners[2:3].repeat(9), owners[3:4].repeat(32), owners[4:5].repeat(62)])
    r2t = torch.cat([r2t, extra])
    r2t = r2t[torch.randperm(r2t.numel(), generator=g)].to(torch.int32)
    Rn = r2t.numel()
    y = W.per_token("randn", 53, 0, Rn, H, torch.bfloat16)
    out0 = W.per_token("randn", 54, 0, T, H, torch.bfloat16)
    ref = R.moe_gather(y, r2t, out0)
    o = out0.clone().to(DEV)
    op.moe_gather(y.to(DEV), r2t.to(DEV), o)
    C.assert_equal(bits(o), bits(ref))


def test_gather_linearity_at_full_size(op):
    """Configuration 3 sizes (65536 rows x 7168): gathering ones with unit weights counts the rows of every token;
    the weighted gather of a constant equals the sum of the token's weights; scatter's permutation is a bijection."""
    T, H, E, k = 8192, 7168, 256, 8
    d = W.router_inputs(T, E, gen_device=DEV)
    w = torch.empty(T, k, device=DEV); ids = torch.empty(T, k, dtype=torch.int32, device=DEV)
    op.fused_moe_gate_deepseek(d["logits"], d["bias"], w, ids, k, True, 8, 4, None, 2.5, 0)
    hid = W.per_token("randn", 21, 0, T, H, torch.bfloat16, gen_device=DEV)
    Rn = T * k
    rows = torch.empty(Rn, H, dtype=torch.int8, device=DEV); sc = torch.empty(Rn, device=DEV)
    r2t = torch.empty(Rn, dtype=torch.int32, device=DEV); cnt = torch.empty(E, dtype=torch.int32, device=DEV)
    st = torch.empty(E, dtype=torch.int32, device=DEV); t2r = torch.empty(T, k, dtype=torch.int32, device=DEV)
    op.moe_scatter_dynamic_quant(hid, ids, w, torch.ones(E, H, device=DEV), rows, sc, r2t, cnt, st, E, 0, 0, t2r)
    assert int(cnt.sum()) == Rn and torch.equal(st, (torch.cumsum(cnt, 0) - cnt).int())
    assert torch.equal(torch.bincount(ids.reshape(-1).long(), minlength=E).int(), cnt)
    assert torch.equal(torch.sort(t2r.reshape(-1)).values, torch.arange(Rn, dtype=torch.int32, device=DEV))
    assert torch.equal(r2t[t2r.reshape(-1).long()], torch.arange(T, device=DEV).repeat_interleave(k).int())
    seg = torch.repeat_interleave(torch.arange(E, device=DEV), cnt.long())
    assert torch.equal(seg.int(), ids.reshape(-1)[torch.argsort(t2r.reshape(-1))])       # rows grouped by expert
    tok_sorted = r2t.long()
    assert bool(((tok_sorted[1:] > tok_sorted[:-1]) | (seg[1:] != seg[:-1])).all())       # ascending tokens inside an expert
    assert int(rows.to(torch.int16).abs().amax(1).min()) == 127                           # every row spans the code range
    ones = torch.ones(Rn, H, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    op.moe_gather(ones, r2t, out)
    assert bool((out == float(k)).all())
    op.moe_gather_weighted(ones, r2t, ids, w, st, out, False, t2r)
    assert torch.allclose(out.float(), w.sum(-1, keepdim=True).expand(T, H), rtol=1e-2)


def test_scatter_config5_full_size_properties(op):
    """Configuration 5 sizes (262,144 tokens x 7168, top-2 of 8: 524,288 rows, 512 tiles - the separate scan kernel):
    the permutation is a bijection ordered by (expert, token), counts equal the histogram of the ids, every row spans
    the code range, and de-quantised rows reproduce (x * w) * smooth to half a quantisation step (sampled rows)."""
    T, H, E, k = 262144, 7168, 8, 2
    logits = W.router_inputs(T, E, gen_device=DEV)["logits"]
    w = torch.empty(T, k, device=DEV); ids = torch.empty(T, k, dtype=torch.int32, device=DEV)
    op.moe_softmax_topk(w, ids, logits, True)
    hid = W.per_token("randn", 21, 0, T, H, torch.bfloat16, gen_device=DEV)
    smooth = 0.5 + torch.rand(E, H, device=DEV)
    Rn = T * k
    rows = torch.empty(Rn, H, dtype=torch.int8, device=DEV); sc = torch.empty(Rn, device=DEV)
    r2t = torch.empty(Rn, dtype=torch.int32, device=DEV); cnt = torch.empty(E, dtype=torch.int32, device=DEV)
    st = torch.empty(E, dtype=torch.int32, device=DEV); t2r = torch.empty(T, k, dtype=torch.int32, device=DEV)
    op.moe_scatter_dynamic_quant(hid, ids, w, smooth, rows, sc, r2t, cnt, st, E, 0, 0, t2r)
    assert int(cnt.sum()) == Rn and torch.equal(st, (torch.cumsum(cnt, 0) - cnt).int())
    assert torch.equal(torch.bincount(ids.reshape(-1).long(), minlength=E).int(), cnt)
    flat = t2r.reshape(-1)
    assert torch.equal(torch.sort(flat).values, torch.arange(Rn, dtype=torch.int32, device=DEV))
    assert torch.equal(r2t[flat.long()], torch.arange(T, device=DEV).repeat_interleave(k).int())
    seg = torch.repeat_interleave(torch.arange(E, device=DEV), cnt.long())
    assert torch.equal(seg.int(), ids.reshape(-1)[torch.argsort(flat)])
    tok = r2t.long()
    assert bool(((tok[1:] > tok[:-1]) | (seg[1:] != seg[:-1])).all())
    sample = torch.randint(0, Rn, (4096,), device=DEV, generator=torch.Generator(device=DEV).manual_seed(0))
    srows = rows[sample].float()
    assert int(srows.abs().amax(1).min()) == 127
    t_of = r2t[sample].long(); e_of = seg[sample]
    slot = (ids[t_of] == e_of.int().unsqueeze(1)).float().argmax(1)
    v = hid[t_of].float() * w[t_of, slot].unsqueeze(1) * smooth[e_of]
    err = (srows * sc[sample].unsqueeze(1) - v).abs()
    assert bool((err <= sc[sample].unsqueeze(1) * (0.5 + 1e-3) + 1e-12).all())
    assert torch.allclose(sc[sample], v.abs().amax(1) / 127.0, rtol=1e-6)


def test_c_abi_dispatch_called_directly(op):
    from mcoplib_b200 import cabi
    from tests.gpu_util import stream_ptr
    lib = cabi.load()
    T, H, E, k = 520, 1024, 8, 2
    w, ids = R.moe_softmax_topk(W.router_inputs(T, E)["logits"], k)
    d = W.dispatch_inputs(T, H, E, k)
    ref = R.moe_scatter_dynamic_quant(d["hidden"], ids, w, d["smooth"], E)
    hg, ig, wg, sg = d["hidden"].to(DEV), ids.to(DEV), w.to(DEV), d["smooth"].to(DEV)
    Rn = T * k
    rows = torch.empty(Rn, H, dtype=torch.int8, device=DEV); sc = torch.empty(Rn, device=DEV); r2t = torch.empty(Rn, dtype=torch.int32, device=DEV)
    cnt = torch.empty(E, dtype=torch.int32, device=DEV); st = torch.empty(E, dtype=torch.int32, device=DEV)
    nbytes = lib.mcop_moe_scatter_workspace_bytes(T, k, E)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    assert lib.mcop_moe_scatter_quant_i8(hg.data_ptr(), ig.data_ptr(), wg.data_ptr(), sg.data_ptr(), rows.data_ptr(), sc.data_ptr(),
                                         r2t.data_ptr(), cnt.data_ptr(), st.data_ptr(), None, T, H, k, E, ws.data_ptr(), nbytes - 16,
                                         stream_ptr()) == -3                      # workspace too small: rejected, nothing launched
    cabi.check(lib.mcop_moe_scatter_quant_i8(hg.data_ptr(), ig.data_ptr(), wg.data_ptr(), sg.data_ptr(), rows.data_ptr(), sc.data_ptr(),
                                             r2t.data_ptr(), cnt.data_ptr(), st.data_ptr(), None, T, H, k, E, ws.data_ptr(), nbytes,
                                             stream_ptr()), lib)
    torch.cuda.synchronize()
    C.assert_equal(r2t, ref[2]); C.assert_equal(cnt, ref[3]); C.assert_codes(rows, ref[0])
    y = d["y"].to(DEV); out = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    gbytes = lib.mcop_moe_gather_workspace_bytes(T, Rn)
    gws = torch.empty(gbytes, dtype=torch.uint8, device=DEV)
    cabi.check(lib.mcop_moe_gather(y.data_ptr(), r2t.data_ptr(), out.data_ptr(), None, 0, T, Rn, H, gws.data_ptr(), gbytes, stream_ptr()), lib)
    torch.cuda.synchronize()
    C.assert_equal(bits(out), bits(R.moe_gather(d["y"], ref[2], torch.zeros(T, H, dtype=torch.bfloat16))))
