"""Generate the golden vectors under tests/golden/ from the reference's OWN torch-native test
references.  Run once, in a container that has the MetaX-MACA/mcoplib checkout:

    python tests/golden/make_golden.py --reference /path/to/mcoplib

The reference's test files cannot be imported (they import the built `mcoplib` extension and
allocate on "cuda"), so each reference function is located by name with `ast`, its source text is
taken from the reference file at run time, and it is executed here on CPU tensors.  No reference
source is stored in this repository: only seeded inputs and the outputs those functions produced.

Two kinds of record are written into golden.npz:
  * "ref:<file>:<function>"  - produced by a function object compiled from the reference file;
  * "formula:<file>:<lines>" - the reference holds the check only as inline statements of a GPU
    runner (or calls a third-party function: vLLM's RMSNorm.forward_native); the same torch
    statements are restated below, next to the citation, and executed.
bf16 tensors are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import argparse
import ast
import os
import textwrap
import types
import typing

import numpy as np
import torch
import torch.nn.functional as F


def _find_def(tree: ast.AST, name: str) -> ast.FunctionDef:
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == name:
            return node
    raise KeyError(name)


def load_function(ref_root: str, rel_path: str, name: str, extra_globals=None, patch=None):
    """Compile function `name` (top-level, method or nested) out of a reference file."""
    path = os.path.join(ref_root, rel_path)
    with open(path, "r", encoding="utf-8") as fh:
        src = fh.read()
    node = _find_def(ast.parse(src), name)
    seg = textwrap.dedent(ast.get_source_segment(src, node))
    if patch:
        for a, b in patch:
            seg = seg.replace(a, b)
    ns = {"torch": torch, "F": F, "np": np, "print": lambda *a, **k: None}
    ns.update(extra_globals or {})
    exec(compile(seg, rel_path, "exec"), ns)
    return ns[name]


def put(store: dict, key: str, **tensors):
    for name, t in tensors.items():
        if isinstance(t, torch.Tensor):
            if t.dtype == torch.bfloat16:
                store[f"{key}/{name}#bf16"] = t.contiguous().view(torch.int16).numpy().view(np.uint16)
            elif t.dtype == torch.float16:
                store[f"{key}/{name}#f16"] = t.contiguous().view(torch.int16).numpy().view(np.uint16)
            else:
                store[f"{key}/{name}"] = t.contiguous().numpy()
        else:
            store[f"{key}/{name}"] = np.asarray(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MCOPLIB_REFERENCE", ""),
                    help="checkout of MetaX-MACA/mcoplib (default: the environment variable MCOPLIB_REFERENCE)")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz"))
    args = ap.parse_args()
    ref = args.reference
    if not ref or not os.path.isdir(ref):
        ap.error("give the reference checkout with --reference or MCOPLIB_REFERENCE")
    store: dict = {}

    # ---------------------------------------------------------------- a11: grouped sigmoid gate
    # unit_test/test_fused_moe_gate_deepseek.py:15-70 biased_grouped_topk, inputs as moe_gate_func
    # (:88-92: torch.rand logits and bias), the three 256-expert cases of TestMoeGate.
    fn = load_function(ref, "unit_test/test_fused_moe_gate_deepseek.py", "biased_grouped_topk")
    for i, (dtype, scaling) in enumerate([(torch.float32, 3.0), (torch.bfloat16, 1.0), (torch.float32, 2.5)]):
        g = torch.Generator().manual_seed(100 + i)
        q_len = 16 if i < 2 else 64
        gating = torch.rand(q_len, 256, generator=g, dtype=torch.float32).to(dtype)
        bias = torch.rand(256, generator=g, dtype=torch.float32).to(dtype)
        if i == 2:  # the BASELINE distribution: logits N(0,1), bias N(0, 0.01)
            gating = torch.randn(q_len, 256, generator=g)
            bias = torch.randn(256, generator=g) * 0.01
        w, ids = fn(gating, gating, bias, 8, True, 8, 4, scaling)
        put(store, f"ref:unit_test/test_fused_moe_gate_deepseek.py:biased_grouped_topk/{i}",
            gating=gating, bias=bias, weights=w, ids=ids, scaling=scaling)

    # ---------------------------------------------------------------- fused_moe_gate_opt ("next" row)
    # unit_test/test_fused_moe_gate_opt.py:78-135 biased_grouped_topk (the -inf masking variant, with the fused
    # shared expert), inputs as moe_gate_func (:152-153: torch.rand logits and bias), TestMoeGate's three cases in
    # bf16 plus fp32 cases (no ties).  With one shared expert the function overwrites the LAST of nine unsorted
    # picks; on the CPU torch.topk returns them in descending order, so the last is the ninth best - checked here.
    fn = load_function(ref, "unit_test/test_fused_moe_gate_opt.py", "biased_grouped_topk", extra_globals={"Optional": typing.Optional})
    cases = [(torch.bfloat16, 256, 8, 4, 8, 0, 1.0), (torch.bfloat16, 160, 1, 1, 8, 0, 1.0), (torch.bfloat16, 160, 1, 1, 9, 1, 1.0),
             (torch.float32, 256, 8, 4, 8, 0, 1.0), (torch.float32, 384, 1, 1, 9, 1, 2.5), (torch.float32, 448, 1, 1, 8, 0, 1.0)]
    for i, (dtype, E, G, TG, k, shared, scaling) in enumerate(cases):
        g = torch.Generator().manual_seed(200 + i)
        gating = torch.rand(16, E, generator=g, dtype=torch.float32).to(dtype)
        bias = torch.rand(E, generator=g, dtype=torch.float32).to(dtype)
        w, ids = fn(gating, gating, bias, k, True, G, TG, shared, scaling)
        if shared:
            assert bool((ids[:, -1] == E).all())
        put(store, f"ref:unit_test/test_fused_moe_gate_opt.py:biased_grouped_topk/{i}", gating=gating, bias=bias, weights=w, ids=ids,
            scaling=scaling, groups=G, topk_group=TG, topk=k, shared=shared)

    # ---------------------------------------------------------------- a4: rms_norm (rms_div form)
    # unit_test/test_rms_norm.py:4-38 rms_norm_ref: after_res / rsqrt(mean+eps) * weight.
    fn = load_function(ref, "unit_test/test_rms_norm.py", "rms_norm_ref")
    g = torch.Generator().manual_seed(7)
    x = torch.randn(8, 1024, generator=g).bfloat16()
    r = torch.randn(8, 1024, generator=g).bfloat16()
    w = (1.0 + 0.1 * torch.randn(1024, generator=g)).bfloat16()
    out, after = fn(x, r, w, None, 1e-6)
    put(store, "ref:unit_test/test_rms_norm.py:rms_norm_ref/0", x=x, residual=r, weight=w, out=out, after_res=after)

    # ---------------------------------------------------------------- head_rms_norm
    # unit_test/test_head_rms_norm.py:4-17 head_rms_norm_ref, applied per head as head_rms_norm_run :21-33.
    fn = load_function(ref, "unit_test/test_head_rms_norm.py", "head_rms_norm_ref")
    g = torch.Generator().manual_seed(42)
    hs = torch.randn(6, 4, 128, generator=g).bfloat16()
    hw = torch.randn(4, 128, generator=g).bfloat16()
    y = hs.clone()
    for h in range(3):
        y[:, h, :] = fn(hs[:, h, :], hw[h, :], 1e-5)
    put(store, "ref:unit_test/test_head_rms_norm.py:head_rms_norm_ref/0", hidden=hs, weight=hw, out=y, head_norm=3)

    # ---------------------------------------------------------------- scale_dynamic_quant
    # unit_test/test_scale_dynamic_quant.py:4-20 scale_dynamic_quant_cpu (+ the known answers :56-60).
    fn = load_function(ref, "unit_test/test_scale_dynamic_quant.py", "scale_dynamic_quant_cpu",
                       patch=[('device="cuda"', 'device="cpu"')])
    g = torch.Generator().manual_seed(13)
    hs = torch.randn(2, 16, 768, generator=g).bfloat16()
    sm = torch.ones(768)
    q, s = fn(hs, sm)
    put(store, "ref:unit_test/test_scale_dynamic_quant.py:scale_dynamic_quant_cpu/0", hidden=hs, smooth=sm, codes=q, scales=s)
    hs = torch.tensor([[[1.0, 2.0, 3.0, 4.0], [4.0, 3.0, 2.0, 1.0]]]).bfloat16()
    sm = torch.tensor([1.0, 1.0, 2.0, 2.0])
    q, s = fn(hs, sm)
    put(store, "ref:unit_test/test_scale_dynamic_quant.py:scale_dynamic_quant_cpu/1", hidden=hs, smooth=sm, codes=q, scales=s)

    # ---------------------------------------------------------------- row quant of a12
    # unit_test/test_moe_swiglu_dq.py:6-14 smooth_per_token_dynamic_quant.
    fn = load_function(ref, "unit_test/test_moe_swiglu_dq.py", "smooth_per_token_dynamic_quant")
    g = torch.Generator().manual_seed(5)
    hs = torch.randn(32, 512, generator=g).bfloat16()
    sm = 0.5 + torch.rand(512, generator=g)
    q, s = fn(hs, sm)
    put(store, "ref:unit_test/test_moe_swiglu_dq.py:smooth_per_token_dynamic_quant/0", hidden=hs, smooth=sm, codes=q, scales=s)

    # ---------------------------------------------------------------- moe_swiglu_dynamic_quantize ("next" row)
    # unit_test/test_moe_swiglu_dq.py:16-44 moe_swiglu_dynamic_quant_run (calls smooth_per_token_dynamic_quant).
    run = load_function(ref, "unit_test/test_moe_swiglu_dq.py", "moe_swiglu_dynamic_quant_run",
                        extra_globals={"smooth_per_token_dynamic_quant": fn})
    g = torch.Generator().manual_seed(6)
    E, H = 4, 256
    counts = torch.tensor([5, 0, 9, 6], dtype=torch.int32)
    starts = (torch.cumsum(counts, 0) - counts).to(torch.int32)
    rows = int(counts.sum())
    xs = torch.randn(rows, 2 * H, generator=g).bfloat16()
    sm = 0.5 + torch.rand(E, H, generator=g)
    qt = torch.zeros(rows, H, dtype=torch.int8)
    st = torch.zeros(rows)
    # the reference function multiplies in bf16 (its inputs are bf16 tensors); feed fp32 views so that it follows
    # the kernel's fp32 arithmetic
    run(xs.float(), sm, counts, starts, qt, st, E)
    put(store, "ref:unit_test/test_moe_swiglu_dq.py:moe_swiglu_dynamic_quant_run/0", x=xs, smooth=sm, counts=counts,
        starts=starts, codes=qt, scales=st)

    # ---------------------------------------------------------------- row quant of fused_silu_mul_dq_* ("next" row)
    # unit_test/test_silu_mul_dq_reorder_mask.py:9-45 as_float32_tensor + ref_dynamic_per_token_quant (the torch part
    # of that test; its SiLU*up product comes from a Triton kernel and cannot run here).  Fed with the fp32 product
    # of the kernel's expression so that it follows the kernel's arithmetic.
    tnames ={"Optional": typing.Optional, "Tuple": typing.Tuple, "Union": typing.Union}
    as32 = load_function(ref, "unit_test/test_silu_mul_dq_reorder_mask.py", "as_float32_tensor",
                         extra_globals=tnames, patch=[("device='cuda'", "device='cpu'")])
    fn = load_function(ref, "unit_test/test_silu_mul_dq_reorder_mask.py", "ref_dynamic_per_token_quant",
                       extra_globals=dict(tnames, as_float32_tensor=as32))
    g = torch.Generator().manual_seed(8)
    gu = torch.randn(24, 2 * 320, generator=g).bfloat16()
    gate, up = gu[:, :320].float(), gu[:, 320:].float()
    v = up * (gate * (1.0 / (1.0 + torch.exp(-gate))))
    q, s = fn(v, torch.int8)
    put(store, "ref:unit_test/test_silu_mul_dq_reorder_mask.py:ref_dynamic_per_token_quant/0", gate_up=gu, product=v,
        codes=q, scales=s.reshape(-1))

    # ---------------------------------------------------------------- a8: store_kv_cache
    # unit_test/test_store_kv.py:91-128 TestKVCacheStorage.run_reference_impl (fp16, seed 42 layout,
    # 8 Q heads / 1 KV head, D 128; token count reduced from 4096 to 48 and two sequences).
    fn = load_function(ref, "unit_test/test_store_kv.py", "run_reference_impl")
    g = torch.Generator().manual_seed(42)
    for i, dtype in enumerate([torch.float16, torch.bfloat16]):
        me = types.SimpleNamespace()
        me.batch_size = 2
        me.q_head_num, me.kv_head_num, me.head_dim = 8, 1 + i, 128
        me.q_lens = [20, 28]
        me.accum_q_lens = [0, 20, 48]
        me.cache_lens = [17, 3]
        me.cache_slot_ids = [1, 0]
        me.dst_type = torch.int8
        total_heads = me.q_head_num + 2 * me.kv_head_num
        me.packed_qkv = torch.randn(48, total_heads, 128, generator=g).to(dtype)
        me.k_scale = torch.randn(me.kv_head_num, 128, generator=g) * 8
        me.v_scale = torch.randn(me.kv_head_num, 128, generator=g) * 8
        me.k_cache = torch.zeros(2, me.kv_head_num, 48, 128, dtype=torch.int8)
        me.v_cache = torch.zeros_like(me.k_cache)
        kc, vc = fn(me)
        put(store, f"ref:unit_test/test_store_kv.py:run_reference_impl/{i}", packed_qkv=me.packed_qkv,
            k_scale=me.k_scale, v_scale=me.v_scale, q_lens=np.array(me.q_lens, np.int32),
            accum_q_lens=np.array(me.accum_q_lens, np.int32), cache_lens=np.array(me.cache_lens, np.int32),
            cache_slot_ids=np.array(me.cache_slot_ids, np.int32), k_cache=kc, v_cache=vc,
            q_head_num=me.q_head_num, kv_head_num=me.kv_head_num)

    # ---------------------------------------------------------------- a6: packed RoPE
    # benchmark/runners/mcoplib_mxbenchmark_rotary_embeding_runners.py:59-81 _torch_rope_impl
    # (cos/sin there are full-D tables with both halves equal to the kernel's half table).
    fn = load_function(ref, "benchmark/runners/mcoplib_mxbenchmark_rotary_embeding_runners.py", "_torch_rope_impl")
    g = torch.Generator().manual_seed(3)
    me = types.SimpleNamespace(q_head_num=4, kv_head_num=2)
    n, D = 24, 128
    packed = torch.randn(n, 8, D, generator=g).bfloat16()
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(64).float().unsqueeze(1) * inv_freq.unsqueeze(0)
    cos_h, sin_h = ang.cos(), ang.sin()
    out = fn(me, packed, torch.cat([cos_h, cos_h], -1), torch.cat([sin_h, sin_h], -1), [n])
    put(store, "ref:benchmark/runners/mcoplib_mxbenchmark_rotary_embeding_runners.py:_torch_rope_impl/0",
        packed_qkv=packed, cos=cos_h, sin=sin_h, out=out, q_head_num=4, kv_head_num=2)

    # ---------------------------------------------------------------- a5: NeoX / GPT-J RoPE
    # benchmark/runners/mcoplib_mxbenchmark_batched_rotary_embedding_runners.py:125-140 apply_rope_ref
    # (nested function; `self.rot_dim` and `half_dim` are its free variables).
    for i, is_neox in enumerate([True, False]):
        me = types.SimpleNamespace(rot_dim=128)
        fn = load_function(ref, "benchmark/runners/mcoplib_mxbenchmark_batched_rotary_embedding_runners.py",
                           "apply_rope_ref", extra_globals={"self": me, "half_dim": 64})
        g = torch.Generator().manual_seed(11 + i)
        n = 20
        q = torch.randn(n, 4, 128, generator=g).bfloat16()
        pos = torch.randint(0, 64, (n,), generator=g)
        cache = torch.cat([cos_h, sin_h], -1)  # fp32 [64, 128]
        rows = cache[pos]
        cos = rows[:, :64].unsqueeze(1)
        sin = rows[:, 64:].unsqueeze(1)
        out = fn(q.float(), cos, sin, is_neox).to(torch.bfloat16)
        put(store, f"ref:benchmark/runners/mcoplib_mxbenchmark_batched_rotary_embedding_runners.py:apply_rope_ref/{i}",
            query=q, positions=pos, cos_sin_cache=cache, out=out, is_neox=int(is_neox))

    # ---------------------------------------------------------------- a2: norm + per-token int8 quant
    # unit_test/test_fused_rms_norm_dq.py:77-117 ref_impl = vLLM RMSNorm.forward_native followed by
    # dynamic per-token int8 quant.  forward_native is third-party (vLLM, the reference targets 0.14.0)
    # and its quant step is a GPU op, so both are restated: forward_native as published
    # (x.float() [+ residual], residual = x.to(dtype), x * rsqrt(mean(x^2)+eps), x.to(dtype) * weight) and
    # the quant as the reference's own check
    # benchmark/runners/mcoplib_mxbenchmark_dynamic_scaled_int8_quant_runners.py:42-62
    # (round(x / scale) clamped to [-128,127], scale = absmax/127).  Shapes/seeds/scaling as :183-199.
    def forward_native(x, weight, eps, residual):
        orig = x.dtype
        x = x.to(torch.float32)
        if residual is not None:
            x = x + residual.to(torch.float32)
            residual = x.to(orig)
        variance = x.pow(2).mean(dim=-1, keepdim=True)
        x = x * torch.rsqrt(variance + eps)
        x = x.to(orig) * weight
        return x, residual

    cases = [(1, 64), (1, 1027), (5, 1033), (4, 2048), (3, 5120), (2, 5137), (4, 4096)]
    for i, (nt, hd) in enumerate(cases):
        for dtype in (torch.bfloat16, torch.float32):
            for add_res in (False, True):
                torch.random.manual_seed(0)
                w = torch.empty(hd, dtype=dtype).normal_(mean=1.0, std=0.1)
                scale = 1 / hd
                if hd == 4096:   # the distribution of BASELINE config 1: x, residual ~ N(0,1)
                    scale = 1.0
                x = torch.randn(nt, hd, dtype=dtype) * scale
                res = torch.randn_like(x) * scale if add_res else None
                n_out, res_out = forward_native(x, w, 1e-6, res)
                nf = n_out.float()
                scales = nf.abs().amax(dim=-1, keepdim=True) / 127.0
                safe = scales.clone()
                safe[safe == 0] = 1.0
                codes = torch.clamp(torch.round(nf / safe), -128, 127).to(torch.int8)
                key = f"formula:unit_test/test_fused_rms_norm_dq.py:77-117/{i}_{str(dtype)[6:]}_{int(add_res)}"
                if hd > 2100 and dtype == torch.float32:
                    continue
                rec = dict(x=x, weight=w, codes=codes, scales=scales)
                if dtype == torch.bfloat16:
                    rec.update(norm=n_out)
                if add_res:
                    rec.update(residual=res, residual_out=res_out)
                put(store, key, **rec)

    # ---------------------------------------------------------------- a1: fused_add_rms_norm
    # benchmark/runners/mcoplib_mxbenchmark_fused_add_rms_norm_runners.py:36-49 (fp32 form, inline).
    g = torch.Generator().manual_seed(21)
    inp = torch.randn(16, 512, generator=g).bfloat16()
    res = torch.randn(16, 512, generator=g).bfloat16()
    w = torch.randn(512, generator=g).bfloat16()
    res_ref = inp.float() + res.float()
    rms = torch.sqrt(res_ref.pow(2).mean(dim=-1, keepdim=True) + 1e-6)
    out_ref = ((res_ref / rms) * w.float()).to(torch.bfloat16)
    put(store, "formula:benchmark/runners/mcoplib_mxbenchmark_fused_add_rms_norm_runners.py:36-49/0",
        x=inp, residual=res, weight=w, out=out_ref, residual_out=res_ref.to(torch.bfloat16))

    # ---------------------------------------------------------------- a10: softmax top-k (sibling op)
    # benchmark/runners/mcoplib_mxbenchmark_topk_softmax_runners.py:38-49: topk(logits) then softmax over
    # the k selected values == renormalised softmax top-k.
    g = torch.Generator().manual_seed(9)
    for i, (N, E, K) in enumerate([(32, 16, 2), (64, 8, 2), (32, 256, 8), (16, 60, 4)]):
        gating = torch.randn(N, E, generator=g)
        vals, idxs = torch.topk(gating.float(), K, dim=-1)
        weights = torch.softmax(vals, dim=-1)
        put(store, f"formula:benchmark/runners/mcoplib_mxbenchmark_topk_softmax_runners.py:38-49/{i}",
            gating=gating, weights=weights, ids=idxs.to(torch.int32), k=K)

    np.savez_compressed(args.out, **store)
    print(f"wrote {args.out}: {len(store)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
