"""Pins the CPU oracle (oracle/ref_ops.py) to the golden vectors that the reference's own
torch-native test references produced (tests/golden/make_golden.py).  Tolerances are the ones the
reference tests use (int8 atol=1, weights 1e-3, ids exact) or tighter."""
import torch

from oracle import ref_ops as R
from oracle.compare import assert_close, assert_codes, assert_equal, code_stats
from tests.golden_io import records


def _gate_tie_rows(r):
    """Rows whose result depends on how exact ties are broken (frequent for bf16 scores): the reference's
    torch function leaves tie order to torch.topk, the kernel contract sends ties to the lower index."""
    score, biased, _, ST = R._gate_scores(r["gating"], r["bias"])
    n = biased.shape[0]
    grp = biased.reshape(n, 8, 32)
    top2 = torch.sort(grp, dim=-1, descending=True).values[..., :2]
    gs = torch.sort(R.rt(top2[..., 0] + top2[..., 1], ST), dim=-1, descending=True).values
    tie = gs[:, 3] == gs[:, 4]
    _, ids, bits = R.fused_moe_gate_deepseek(r["gating"], r["bias"], 8, True, 8, 4, 1.0)
    emask = ((bits.unsqueeze(1) >> torch.arange(8).unsqueeze(0)) & 1).bool().unsqueeze(-1).expand(n, 8, 32).reshape(n, 256)
    srt = torch.sort(torch.where(emask, biased, torch.full_like(biased, -1e30)), dim=-1, descending=True).values
    return tie | (srt[:, 7] == srt[:, 8])


def test_gate_matches_biased_grouped_topk(golden):
    recs = records(golden, "ref:unit_test/test_fused_moe_gate_deepseek.py:biased_grouped_topk")
    assert len(recs) == 3
    for key, r in recs:
        w, ids, _ = R.fused_moe_gate_deepseek(r["gating"], r["bias"], 8, True, 8, 4, r["scaling"])
        keep = ~_gate_tie_rows(r)
        if r["gating"].dtype == torch.float32:
            assert bool(keep.all()), key
        assert int(keep.sum()) * 2 >= keep.numel(), key
        # the reference compares row-sorted ids exactly and row-sorted weights to 1e-3
        # (unit_test/test_fused_moe_gate_deepseek.py:96-103)
        assert_equal(torch.sort(ids, dim=1).values[keep], torch.sort(r["ids"], dim=1).values[keep], key)
        tol = 1e-3 if r["gating"].dtype == torch.float32 else 2e-2   # bf16 weights: one bf16 ulp of 3.0
        assert torch.allclose(torch.sort(w, dim=1).values[keep], torch.sort(r["weights"], dim=1).values[keep],
                              rtol=tol, atol=tol), key
        # ours is additionally ordered by descending biased score
        _, biased, _, _ = R._gate_scores(r["gating"], r["bias"])
        sel = torch.gather(biased, 1, ids.long())
        assert bool((sel[:, :-1] >= sel[:, 1:]).all()), key


def test_rms_norm_div_form(golden):
    (key, r), = records(golden, "ref:unit_test/test_rms_norm.py:rms_norm_ref")
    out, after = R.rms_norm(r["x"], r["weight"], 1e-6, residual=r["residual"], rms_div=True)
    # the reference function adds in bf16 and keeps bf16 intermediates; the kernel works in fp32
    assert_close(out, r["out"], key, rel=2e-2, abs_=2e-2)
    assert_close(after, r["after_res"], key)


def test_head_rms_norm(golden):
    (key, r), = records(golden, "ref:unit_test/test_head_rms_norm.py:head_rms_norm_ref")
    out = R.head_rms_norm(r["hidden"], r["weight"], 1e-5, 0, r["head_norm"])
    assert_close(out, r["out"], key, rel=2e-2, abs_=2e-2)
    assert torch.equal(out[:, r["head_norm"]:], r["hidden"][:, r["head_norm"]:])


def test_scale_dynamic_quant(golden):
    recs = records(golden, "ref:unit_test/test_scale_dynamic_quant.py:scale_dynamic_quant_cpu")
    for key, r in recs:
        q, s = R.scale_dynamic_quant(r["hidden"].reshape(-1, r["hidden"].shape[-1]), r["smooth"])
        assert torch.allclose(s, r["scales"].reshape(-1), rtol=1e-5), key
        assert code_stats(q, r["codes"].reshape(q.shape))["max_abs"] <= 1, key
    # known answers of the reference test (unit_test/test_scale_dynamic_quant.py:56-60)
    r = recs[1][1]
    _, s = R.scale_dynamic_quant(r["hidden"].reshape(-1, 4), r["smooth"])
    assert abs(float(s[0]) - 8.0 / 127) < 1e-5 and abs(float(s[1]) - 4.0 / 127) < 1e-5


def test_scatter_row_quant_matches_smooth_per_token_dynamic_quant(golden):
    (key, r), = records(golden, "ref:unit_test/test_moe_swiglu_dq.py:smooth_per_token_dynamic_quant")
    n = r["hidden"].shape[0]
    # one expert, k = 1, weight 1: every token becomes one row, in token order
    ids = torch.zeros(n, 1, dtype=torch.int32)
    w = torch.ones(n, 1)
    rows, scales, row2tok, counts, starts, tok2row = R.moe_scatter_dynamic_quant(
        r["hidden"], ids, w, r["smooth"].reshape(1, -1), 1)
    assert_equal(row2tok, torch.arange(n, dtype=torch.int32), key)
    assert int(counts[0]) == n and int(starts[0]) == 0
    assert torch.allclose(scales, r["scales"], rtol=1e-5), key
    assert_codes(rows, r["codes"], key, frac=1e-3)


def test_store_kv(golden):
    recs = records(golden, "ref:unit_test/test_store_kv.py:run_reference_impl")
    assert len(recs) == 2
    for key, r in recs:
        kc0 = torch.zeros_like(r["k_cache"])
        kc, vc = R.store_kv_cache(r["packed_qkv"], r["q_lens"], r["accum_q_lens"], r["cache_lens"],
                                  r["cache_slot_ids"], kc0, kc0.clone(), r["k_scale"], r["v_scale"],
                                  r["q_head_num"], r["kv_head_num"])
        # reference tolerance is atol 0.5 (unit_test/test_store_kv.py:156-169): i.e. exact for integers
        assert_equal(kc, r["k_cache"], key + " k")
        assert_equal(vc, r["v_cache"], key + " v")


def test_packed_rope(golden):
    (key, r), = records(golden, "ref:benchmark/runners/mcoplib_mxbenchmark_rotary_embeding_runners.py:_torch_rope_impl")
    n = r["packed_qkv"].shape[0]
    out = R.rotary_embedding_packed(
        r["packed_qkv"], torch.tensor([n], dtype=torch.int32), torch.tensor([0, n], dtype=torch.int32),
        torch.tensor([0], dtype=torch.int32), r["cos"], r["sin"], r["packed_qkv"].clone(),
        r["q_head_num"], r["kv_head_num"])
    assert_equal(out.view(torch.int16), r["out"].view(torch.int16), key)  # same fp32 formula: bit-exact


def test_rope_fp32_cache(golden):
    recs = records(golden, "ref:benchmark/runners/mcoplib_mxbenchmark_batched_rotary_embedding_runners.py:apply_rope_ref")
    assert len(recs) == 2
    for key, r in recs:
        q, _ = R.rotary_embedding(r["positions"], r["query"].reshape(r["query"].shape[0], -1), None, 128,
                                  r["cos_sin_cache"], bool(r["is_neox"]))
        assert_equal(q.reshape(r["out"].shape).view(torch.int16), r["out"].view(torch.int16), key)
        # the bf16-cache contract rounds after every operation: stays within the bf16 tolerance
        qb, _ = R.rotary_embedding(r["positions"], r["query"].reshape(r["query"].shape[0], -1), None, 128,
                                   r["cos_sin_cache"].bfloat16(), bool(r["is_neox"]))
        assert_close(qb.reshape(r["out"].shape), r["out"], key, rel=3e-2, abs_=3e-2)


def test_norm_quant_matches_forward_native_plus_quant(golden):
    recs = records(golden, "formula:unit_test/test_fused_rms_norm_dq.py:77-117")
    assert len(recs) >= 20
    n_diff = n_all = 0
    for key, r in recs:
        q, s, res = R.rms_norm_dynamic_per_token_quant(r["x"], r["weight"], 1e-6, residual=r.get("residual"))
        assert torch.allclose(s, r["scales"]), key           # reference: allclose on scales
        st = code_stats(q, r["codes"])
        assert st["max_abs"] <= 1, (key, st)                 # reference: int8 atol=1
        n_diff += st["n_diff"]
        n_all += st["n"]
        if "residual_out" in r:
            assert torch.equal(res.view(torch.int16) if res.dtype == torch.bfloat16 else res,
                               r["residual_out"].view(torch.int16) if res.dtype == torch.bfloat16 else r["residual_out"]), key
    # x*(1/scale) (kernel form) vs x/scale (test form) may flip a rounding on a few elements only
    assert n_diff / n_all < 1e-3, (n_diff, n_all)


def test_fused_add_rms_norm(golden):
    (key, r), = records(golden, "formula:benchmark/runners/mcoplib_mxbenchmark_fused_add_rms_norm_runners.py:36-49")
    out, res = R.fused_add_rms_norm(r["x"], r["residual"], r["weight"], 1e-6)
    assert_equal(res.view(torch.int16), r["residual_out"].view(torch.int16), key)
    # the runner's reference keeps fp32 throughout; the kernel contract rounds to bf16 twice
    assert_close(out, r["out"], key, rel=2e-2, abs_=2e-2)


def test_softmax_topk(golden):
    recs = records(golden, "formula:benchmark/runners/mcoplib_mxbenchmark_topk_softmax_runners.py:38-49")
    assert len(recs) == 4
    for key, r in recs:
        w, ids = R.moe_softmax_topk(r["gating"], r["k"])
        assert_equal(ids, r["ids"], key)
        assert torch.allclose(w, r["weights"], rtol=1e-5, atol=1e-6), key


def test_dynamic_scaled_int8_quant_against_the_runner_formula():
    # benchmark/runners/mcoplib_mxbenchmark_dynamic_scaled_int8_quant_runners.py:42-62: round(x / scale) clamped
    g = torch.Generator().manual_seed(17)
    x = torch.randn(64, 777, generator=g).bfloat16()
    x[5] = 0
    q, s = R.dynamic_scaled_int8_quant(x)
    safe = s.clone()
    safe[safe == 0] = 1.0
    ref = torch.clamp(torch.round(x.float() / safe), -128, 127).to(torch.int8)
    assert code_stats(q, ref)["max_abs"] <= 1
    assert code_stats(q, ref)["frac_diff"] < 1e-3
    assert int(q[5].abs().max()) == 0 and float(s[5]) == 0.0
