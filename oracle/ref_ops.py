"""CPU restatement of the mcoplib per-token inference hot path.  TEST INFRASTRUCTURE ONLY.

This module is the parity oracle: tests, the smoke check and the CPU-baseline leg of the
benchmark may call it; nothing in the shipped package imports it.  Every function restates,
in plain torch on CPU tensors, the arithmetic sequence (including every intermediate rounding)
of one reference operator.  Citations are paths inside the MetaX-MACA/mcoplib tree.

Pinning status (see tests/golden): the functions below are checked against golden vectors
produced by the reference's own torch-native test references for rms_norm_dynamic_per_token_quant
(unit_test/test_fused_rms_norm_dq.py), fused_add_rms_norm (benchmark runner), rms_norm
(unit_test/test_rms_norm.py), NeoX RoPE (benchmark runners), store_kv_cache
(unit_test/test_store_kv.py), reshape_and_cache_flash (benchmark runner), softmax top-k
(benchmark runner of the sibling op), fused_moe_gate_deepseek
(unit_test/test_fused_moe_gate_deepseek.py) and the smooth per-token quant
(unit_test/test_moe_swiglu_dq.py).  No reference test asserts values for the 9-argument
fused_rms_norm_dq, moe_scatter_dynamic_quant or moe_gather: for those three the oracle is a
restatement of the cited kernel lines only ("parity unpinned").

Conventions: `T` is the activation dtype (bf16 unless stated).  `rt(v, T)` rounds an fp32
tensor to T (round-to-nearest-even) and returns it widened back to fp32.  int8 conversion is
round-half-even (torch.round) followed by the clamp each reference kernel applies.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

FLT_EPSILON = float(torch.finfo(torch.float32).eps)


def rt(v: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round an fp32 tensor to `dtype` and widen back to fp32."""
    if dtype == torch.float32:
        return v.float()
    return v.to(dtype).float()


def _rsqrt(v: torch.Tensor) -> torch.Tensor:
    # 1/sqrt(v) with IEEE division and square root, the form CPU torch evaluates.
    return 1.0 / torch.sqrt(v)


def _mean_sq(s: torch.Tensor) -> torch.Tensor:
    """mean(s^2) over the last dim as the correctly rounded fp32 value (accumulated in float64): the result
    every fp32 summation order of the reference kernels approximates, and independent of any order."""
    return (s.double() * s.double()).mean(dim=-1, keepdim=True).float()


# --------------------------------------------------------------------------------------
# Part 1: residual add + RMSNorm (+ per-token int8 quant)
# --------------------------------------------------------------------------------------

def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                       eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """op/vllm/layernorm_kernels.cu:92-144 (vector form) and :150-182 (scalar form),
    arithmetic of op/vllm/type_convert.cuh:104-165.

    r = T(x + res); res := r; var = mean(float(r)^2); out = T(T(float(r) * rsqrt(var+eps)) * w).
    Returns (out, new_residual) in T."""
    T = x.dtype
    r = rt(x.float() + residual.float(), T)
    var = _mean_sq(r)
    inv = _rsqrt(var + eps)
    n = rt(rt(r * inv, T) * weight.float(), T)
    return n.to(T), r.to(T)


def rms_norm_dynamic_per_token_quant(
        x: torch.Tensor, weight: torch.Tensor, eps: float,
        residual: Optional[torch.Tensor] = None,
        scale_ub: Optional[torch.Tensor] = None,
        return_norm: bool = False,
):
    """op/vllm/quantization/fused_kernels/fused_layernorm_dynamic_per_token_quant.cu:14-90 with
    layernorm_utils.cuh:17-45 (rms), :145-177 (scale) and :180-217 (norm + quant);
    same contract as mcoplib.op.rms_norm_dynamic_per_token_quant_custom
    (op/rms_norm_dynamic_per_token_quant.cu:94-186).

    s = float(x) + float(res); res := T(s); var = mean(s^2) on the unrounded s;
    n = T(T(s * rsqrt(var+eps)) * w); a = max|n| (clamped by scale_ub if given);
    scale = max(a / 127, FLT_EPSILON); q = clamp(rne(n * (1/scale)), -128, 127).
    Returns (codes int8 [T,H], scales fp32 [T,1], new_residual or None); with return_norm also n in T, the extra
    out_bf16 output of sglang's flavour (op/sglang/csrc/elementwise/fused_layernorm_dynamic_per_token_quant_custom.cu:434-460,
    norm_and_quant in op/sglang/include/layernorm_utils.cuh)."""
    T = x.dtype
    s = x.float()
    new_res = None
    if residual is not None:
        s = s + residual.float()
        new_res = s.to(T)
    var = _mean_sq(s)
    inv = _rsqrt(var + eps)
    n = rt(rt(s * inv, T) * weight.float(), T)
    a = n.abs().amax(dim=-1, keepdim=True)
    if scale_ub is not None:
        a = torch.minimum(a, scale_ub.float().reshape(()))
    scale = torch.clamp(a / 127.0, min=FLT_EPSILON)
    q = torch.round(n * (1.0 / scale)).clamp(-128, 127).to(torch.int8)
    if return_norm:
        return q, scale.reshape(-1, 1), new_res, n.to(T)
    return q, scale.reshape(-1, 1), new_res


def fused_add_rms_norm_dynamic_per_token_quant_padding_output(
        x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, pad_size: int, eps: float, form: int = 0):
    """mcoplib.op.fused_add_rms_norm_dynamic_per_token_quant_padding_output (wrapper mcoplib/custom_ops.py:7-27),
    op/fused_add_layernorm_per_token_quant_padding_output.cu.  PARITY UNPINNED: the reference test
    (unit_test/test_fused_add_rms_norm_custom.py:41-46) evaluates allclose without asserting it.

    The reference picks one of two arithmetic forms by the row length (:371-394); form 0 = its choice.
      form 1 (hidden == 7168, kernel :182-283): s = float(x) + float(res); res := T(s); v = s * float(w);
        a = max|v|; r = rsqrt(mean(s^2) + eps); scale = max(a * r / 127, FLT_EPSILON); y = v * r; norm = T(y);
        code = clamp(rne(y * (1/scale)), -128, 127).
      form 2 (other lengths, kernel :287-340): a = max|T(T(s) * w)|; r from the unrounded s; scale as above;
        n = T(T(float(T(s)) * r) * w); code = clamp(rne(float(n) * (1/scale)), -128, 127); norm = n.
    Record of a token: pad_size elements of T = bytes [0, H) codes, [H, H+4) the fp32 scale, rest not written.
    Returns (packed uint8 [T, 2*pad_size] with unwritten bytes 0, new_residual T, norm T, codes int8, scales fp32 [T,1])."""
    T = x.dtype
    Tn, H = x.shape
    if form == 0:
        form = 1 if H == 7168 else 2
    s = x.float() + residual.float()
    new_res = s.to(T)
    inv = _rsqrt(_mean_sq(s) + eps)
    w = weight.float()
    if form == 1:
        v = s * w
        a = v.abs().amax(dim=-1, keepdim=True)
        y = v * inv
        norm = y.to(T)
    else:
        a = rt(rt(s, T) * w, T).abs().amax(dim=-1, keepdim=True)
        y = rt(rt(rt(s, T) * inv, T) * w, T)
        norm = y.to(T)
    scale = torch.clamp((a * inv) / 127.0, min=FLT_EPSILON)
    q = torch.round(y * (1.0 / scale)).clamp(-128, 127).to(torch.int8)
    packed = torch.zeros(Tn, 2 * pad_size, dtype=torch.uint8)
    packed[:, :H] = q.view(torch.uint8)
    packed[:, H:H + 4] = scale.reshape(-1).contiguous().view(torch.uint8).reshape(Tn, 4)
    return packed, new_res, norm, q, scale.reshape(-1, 1)


def fused_rms_norm_dq(
        x: torch.Tensor, weight: torch.Tensor, smooth: torch.Tensor, eps: float,
        residual: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """9-argument mcoplib.op.rms_norm_dynamic_per_token_quant, op/fused_rms_norm_dq.cu:69-186,
    :226-303.  PARITY UNPINNED (no reference test asserts its values).

    The reference DIVIDES by rsqrt(mean+eps) (lines 139, 179), i.e. multiplies by the root
    mean square; that literal convention is kept.
    s = float(x) + float(res); after_res = T(s); var = mean(s^2) (unrounded s);
    r = rsqrt(var+eps); a = float(after_res); after_norm = T(a / r * w);
    y = a / r * w * smooth; scale = max|y| / 127; q = clamp(rne(y * (1/scale)), -128, 127)
    (op/fused_rms_norm_dq.cu:54-66 and the conversion in kernel/utils.cuh).
    Returns (codes, scales [T,1], after_res, after_norm)."""
    T = x.dtype
    s = x.float()
    if residual is not None:
        s = s + residual.float()
    after_res = s.to(T)
    var = _mean_sq(s)
    r = _rsqrt(var + eps)
    a = after_res.float()
    nw = a / r * weight.float()
    after_norm = nw.to(T)
    y = nw * smooth.float()
    scale = (y.abs().amax(dim=-1, keepdim=True).double() / 127.0).float()
    inv = 1.0 / scale
    q = torch.nan_to_num(torch.round(y * inv), nan=0.0).clamp(-127, 127).to(torch.int8)
    return q, scale.reshape(-1, 1), after_res, after_norm


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float,
             residual: Optional[torch.Tensor] = None, rms_div: bool = False,
             ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """mcoplib.op.rms_norm, op/fused_rms_norm_dq.cu:305-386 (and :980-999).

    s = float(x) [+ float(res)], after_res = T(s); r = rsqrt(mean(s^2)+eps);
    d = (1/r) if rms_div else r; out = T(s * d * w) with one rounding."""
    T = x.dtype
    s = x.float()
    after_res = None
    if residual is not None:
        s = s + residual.float()
        after_res = s.to(T)
    var = _mean_sq(s)
    r = _rsqrt(var + eps)
    d = (1.0 / r) if rms_div else r
    out = (s * d * weight.float()).to(T)
    return out, after_res


def head_rms_norm(hidden: torch.Tensor, weight: torch.Tensor, eps: float, head_offset: int,
                  head_norm: int) -> torch.Tensor:
    """mcoplib.op.head_rms_norm, op/fused_rms_norm_dq.cu:493-557,804-812: per-head norm of heads
    [head_offset, head_offset+head_norm) of hidden [T, heads, D]; out = T(x / rsqrt(mean+eps) * w[h])
    (the same divide-by-rsqrt convention, unit_test/test_head_rms_norm.py:4-17); other heads are
    left as they are in the returned copy."""
    T = hidden.dtype
    out = hidden.clone()
    sel = hidden[:, head_offset:head_offset + head_norm, :].float()
    var = _mean_sq(sel)
    r = _rsqrt(var + eps)
    w = weight.float().reshape(-1, hidden.shape[-1])[head_offset:head_offset + head_norm]
    out[:, head_offset:head_offset + head_norm, :] = (sel / r * w.unsqueeze(0)).to(T)
    return out


def scale_dynamic_quant(hidden: torch.Tensor, smooth: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """mcoplib.op.scale_dynamic_quant, op/scale_dynamic_quant.cu:40-125:
    y = float(x) * smooth; scale = max|y| / 127; q = clamp(rne(y / scale), -128, 127).
    Returns (codes int8, scales fp32 [T])."""
    y = hidden.float() * smooth.float()
    scale = y.abs().amax(dim=-1, keepdim=True) / 127.0
    q = torch.nan_to_num(torch.round(y / scale), nan=0.0).clamp(-128, 127).to(torch.int8)
    return q, scale.reshape(-1)


def dynamic_scaled_int8_quant(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """torch.ops._C.dynamic_scaled_int8_quant, symmetric form,
    op/vllm/quantization/compressed_tensors/int8_quant_kernels.cu:95-132: scale = max|x| / 127;
    q = clamp(rne(float(x) * (127 / max|x|)), -128, 127), inv = 0 for an all-zero row.
    Pinned by the reference's own check round(x / scale)
    (benchmark/runners/mcoplib_mxbenchmark_dynamic_scaled_int8_quant_runners.py:42-62), tolerance 1 code.
    Returns (codes int8, scales fp32 [tokens, 1])."""
    f = x.float()
    a = f.abs().amax(dim=-1, keepdim=True)
    # tensor / tensor: a correctly rounded division (scalar / tensor is evaluated by torch as reciprocal * scalar)
    inv = torch.where(a == 0, torch.zeros_like(a), torch.full_like(a, 127.0) / a)
    q = torch.round(f * inv).clamp(-128, 127).to(torch.int8)
    return q, (a / 127.0).reshape(-1, 1)


# --------------------------------------------------------------------------------------
# Part 2: RoPE and the int8 KV store
# --------------------------------------------------------------------------------------

def _rope_pair(x: torch.Tensor, y: torch.Tensor, c: torch.Tensor, s: torch.Tensor,
               T: torch.dtype, per_op_rounding: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    if per_op_rounding:
        # arithmetic in T: every product and the sum/difference are rounded to T
        # (op/vllm/pos_encoding_kernels.cu:32-35)
        xo = rt(rt(x * c, T) - rt(y * s, T), T)
        yo = rt(rt(y * c, T) + rt(x * s, T), T)
    else:
        # fp32 arithmetic, one rounding at the store (op/rotary_embedding.cu:11-28)
        xo = rt(x * c - y * s, T)
        yo = rt(y * c + x * s, T)
    return xo, yo


def _rotate_heads(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot_dim: int,
                  is_neox: bool, per_op_rounding: bool) -> torch.Tensor:
    """t: [N, heads, D] in T; cos, sin: fp32 [N, rot_dim/2] (already widened)."""
    T = t.dtype
    out = t.clone()
    half = rot_dim // 2
    f = t.float()
    c = cos.unsqueeze(1)
    s = sin.unsqueeze(1)
    if is_neox:
        x = f[..., :half]
        y = f[..., half:rot_dim]
        xo, yo = _rope_pair(x, y, c, s, T, per_op_rounding)
        out[..., :half] = xo.to(T)
        out[..., half:rot_dim] = yo.to(T)
    else:
        x = f[..., 0:rot_dim:2]
        y = f[..., 1:rot_dim:2]
        xo, yo = _rope_pair(x, y, c, s, T, per_op_rounding)
        out[..., 0:rot_dim:2] = xo.to(T)
        out[..., 1:rot_dim:2] = yo.to(T)
    return out


def rotary_embedding(positions: torch.Tensor, query: torch.Tensor, key: Optional[torch.Tensor],
                     head_size: int, cos_sin_cache: torch.Tensor, is_neox: bool,
                     ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """torch.ops._C.rotary_embedding, op/vllm/pos_encoding_kernels.cu:12-102.

    cos_sin_cache [max_pos, rot_dim] = cos(rot_dim/2) || sin(rot_dim/2).  With a cache in the
    activation dtype the arithmetic is carried out in T (per-operation rounding, lines 32-35).
    With an fp32 cache (extension of this build) the arithmetic is fp32 with a single rounding,
    the contract of mcoplib.op.rotary_embedding (op/rotary_embedding.cu:11-28).
    Returns rotated copies (query', key')."""
    n = positions.numel()
    rot_dim = cos_sin_cache.shape[-1]
    half = rot_dim // 2
    rows = cos_sin_cache[positions.reshape(-1).long()]
    per_op = cos_sin_cache.dtype != torch.float32
    cos = rows[:, :half].float()
    sin = rows[:, half:].float()
    q = _rotate_heads(query.reshape(n, -1, head_size), cos, sin, rot_dim, is_neox, per_op).reshape(query.shape)
    k = None
    if key is not None:
        k = _rotate_heads(key.reshape(n, -1, head_size), cos, sin, rot_dim, is_neox, per_op).reshape(key.shape)
    return q, k


def token_positions(accum_q_lens: torch.Tensor, cache_lens: torch.Tensor, num_tokens: int) -> torch.Tensor:
    """Position of every packed token: cache_lens[b] + (t - accum_q_lens[b]) for the sequence b
    that holds token t (op/rotary_embedding.cu:31-38,72-77)."""
    accum = accum_q_lens.long()
    t = torch.arange(num_tokens)
    b = torch.searchsorted(accum[1:].contiguous(), t, right=True)
    return cache_lens.long()[b] + (t - accum[b])


def rotary_embedding_packed(packed_qkv: torch.Tensor, q_len: torch.Tensor, accum_q_lens: torch.Tensor,
                            cache_lens: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                            output: torch.Tensor, q_head_num: int, kv_head_num: int) -> torch.Tensor:
    """mcoplib.op.rotary_embedding, op/rotary_embedding.cu:11-121.  PARITY of values unpinned by a
    reference assertion; the formula is pinned through the benchmark runner's torch form.

    packed [T, Hq+2Hkv, D]; cos/sin fp32 [max_pos, D/2]; NeoX pairs; fp32 math, one rounding;
    writes the Q and K heads of a copy of `output`, leaving its V heads untouched."""
    n = packed_qkv.shape[0]
    pos = token_positions(accum_q_lens, cache_lens, n)
    out = output.clone()
    nqk = q_head_num + kv_head_num
    D = packed_qkv.shape[-1]
    rot = _rotate_heads(packed_qkv[:, :nqk, :], cos[pos].float(), sin[pos].float(), D, True, False)
    out[:, :nqk, :] = rot
    return out


def fused_rope_fwd(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   indexes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """mcoplib.op.fused_rope_fwd, kernel/fused_rope_kernel.h:6-96: NeoX RoPE on the Q and K planes
    of [S, 3, H, D]; cos/sin [*, D/2] in T, widened to fp32; fp32 math, one rounding."""
    S = qkv.shape[0]
    idx = torch.arange(S) if indexes is None else indexes.long()
    D = qkv.shape[-1]
    out = qkv.clone()
    c = cos.reshape(-1, D // 2)[idx].float()
    s = sin.reshape(-1, D // 2)[idx].float()
    for plane in (0, 1):
        out[:, plane] = _rotate_heads(qkv[:, plane], c, s, D, True, False)
    return out


def fused_rope_bwd(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   indexes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """mcoplib.op.fused_rope_bwd, kernel/fused_rope_kernel.h:101-191: the transposed rotation,
    x' = x*c + y*s, y' = -x*s + y*c (lines 172-176), fp32 math, one rounding.  Negating the sine is
    exact, so this is the forward formula evaluated with -sin."""
    return fused_rope_fwd(qkv, cos, -sin, indexes)


def float_to_int8_sym(v: torch.Tensor) -> torch.Tensor:
    """kernel/utils.h:219-226: round-half-even, clamp to [-127, 127]; NaN converts to 0."""
    return torch.nan_to_num(torch.round(v), nan=0.0).clamp(-127, 127).to(torch.int8)


def store_kv_cache(packed_qkv: torch.Tensor, q_lens, accum_q_lens, cache_lens, cache_slot_ids,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, k_scale: torch.Tensor,
                   v_scale: torch.Tensor, q_head_num: int, kv_head_num: int,
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """mcoplib.op.store_kv_cache_cuda_interface, op/store_kv.cu:145-218.

    code = clamp(rne(float(x) * scale[h, d]), -127, 127); scale tensors [Hkv, D] are multipliers;
    destination cache[slot, h, cache_len + i, :] of an int8 cache [slots, Hkv, max_len, D]."""
    kc = k_cache.clone()
    vc = v_cache.clone()
    for b in range(len(q_lens)):
        ql = int(q_lens[b]); off = int(accum_q_lens[b]); cl = int(cache_lens[b]); slot = int(cache_slot_ids[b])
        k = packed_qkv[off:off + ql, q_head_num:q_head_num + kv_head_num].float()
        v = packed_qkv[off:off + ql, q_head_num + kv_head_num:q_head_num + 2 * kv_head_num].float()
        kc[slot, :, cl:cl + ql] = float_to_int8_sym(k * k_scale.float().unsqueeze(0)).transpose(0, 1)
        vc[slot, :, cl:cl + ql] = float_to_int8_sym(v * v_scale.float().unsqueeze(0)).transpose(0, 1)
    return kc, vc


def reshape_and_cache_flash(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                            value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """torch.ops._C_cache_ops.reshape_and_cache_flash with kv_cache_dtype "auto",
    op/vllm/cache_kernels.cu:193-266: blk = slot / block_size, off = slot % block_size,
    negative slots are skipped; cache [num_blocks, block_size, Hkv, D]."""
    kc = key_cache.clone()
    vc = value_cache.clone()
    bs = kc.shape[1]
    slots = slot_mapping.long()
    keep = slots >= 0
    blk = torch.div(slots[keep], bs, rounding_mode="floor")
    off = slots[keep] % bs
    kc[blk, off] = key.reshape(key.shape[0], kc.shape[2], kc.shape[3])[keep].to(kc.dtype)
    vc[blk, off] = value.reshape(value.shape[0], vc.shape[2], vc.shape[3])[keep].to(vc.dtype)
    return kc, vc


def reshape_and_cache(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                      slot_mapping: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """torch.ops._C_cache_ops.reshape_and_cache with kv_cache_dtype "auto", op/vllm/cache_kernels.cu:133-190:
    key_cache [num_blocks, H, D/x, block_size, x], value_cache [num_blocks, H, D, block_size];
    blk = slot / block_size, off = slot % block_size, negative slots are skipped;
    key_cache[blk, h, g, off, i] = key[t, h, g*x + i], value_cache[blk, h, d, off] = value[t, h, d]."""
    kc = key_cache.clone()
    vc = value_cache.clone()
    nb, H, G, bs, x = kc.shape
    slots = slot_mapping.long()
    keep = slots >= 0
    blk = torch.div(slots[keep], bs, rounding_mode="floor")
    off = slots[keep] % bs
    n = key.shape[0]
    k = key.reshape(n, H, G, x)[keep].to(kc.dtype)
    v = value.reshape(n, H, G * x)[keep].to(vc.dtype)
    kc[blk, :, :, off, :] = k
    vc[blk, :, :, off] = v
    return kc, vc


def rope_kv_store_int8(positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                       head_size: int, cos_sin_cache: torch.Tensor, is_neox: bool,
                       key_cache: torch.Tensor, value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                       k_scale: torch.Tensor, v_scale: torch.Tensor):
    """Fused RoPE + int8 paged KV store.  No single reference operator does this; it is the
    composition rotary_embedding (above) -> quantise the ROUNDED rotated K and the V with
    code = clamp(rne(float(v) * (1/scale[h])), -127, 127) (store_kv arithmetic with a per-head
    dequantisation scale) -> paged addressing of reshape_and_cache_flash.
    Returns (query', key', key_cache', value_cache')."""
    q, k = rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox)
    n = key.shape[0]
    Hkv = key_cache.shape[2]
    inv_k = (1.0 / k_scale.float()).reshape(1, Hkv, 1)
    inv_v = (1.0 / v_scale.float()).reshape(1, Hkv, 1)
    kq = float_to_int8_sym(k.reshape(n, Hkv, head_size).float() * inv_k)
    vq = float_to_int8_sym(value.reshape(n, Hkv, head_size).float() * inv_v)
    kc, vc = reshape_and_cache_flash(kq, vq, key_cache, value_cache, slot_mapping)
    return q, k, kc, vc


# --------------------------------------------------------------------------------------
# Part 3: routing, dispatch, combine
# --------------------------------------------------------------------------------------

def stable_topk(scores: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k along the last dim in descending order with ties going to the LOWEST index."""
    order = torch.sort(scores, dim=-1, descending=True, stable=True)
    return order.values[..., :k], order.indices[..., :k]


def moe_softmax_topk(gating: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """mcoplib.op.moe_softmax_topk, kernel/moe_softmax_topk.cuh:917-1041.  PARITY UNPINNED for the
    op itself; the math (renormalised softmax top-k) is pinned through the sibling op's benchmark check.

    p = exp(x - max) * (1 / sum exp(x - max)); k rounds of arg-max on p, ties to the lowest index,
    output in descending order; weights = p_sel / (p_sel summed in selection order).
    The per-row (not per-warp) result is produced for every E (the reference aliases rows when E <= 32)."""
    x = gating.float()
    e = torch.exp(x - x.amax(dim=-1, keepdim=True))
    p = e * (1.0 / e.sum(dim=-1, keepdim=True))
    vals, ids = stable_topk(p, k)
    tot = torch.zeros(vals.shape[:-1], dtype=torch.float32)
    for j in range(k):
        tot = tot + vals[..., j]
    return vals / tot.unsqueeze(-1), ids.to(torch.int32)


def topk_softmax(gating: torch.Tensor, k: int, renormalize: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """torch.ops._moe_C.topk_softmax, op/vllm/moe/topk_softmax_kernels.cu:396-545 (topkGatingSoftmax) and :884-918.
    Pinned by the check of benchmark/runners/mcoplib_mxbenchmark_topk_softmax_runners.py:38-49 (topk of the logits,
    softmax over the selected = the renormalised form; ids exact).

    Logits of any float type are widened to fp32; p = exp(x - max) * (1 / sum); k rounds of arg-max, ties to the
    lowest index; weights = p_sel, divided by their sum (accumulated in selection order, 1 if it is 0) only when
    renormalize.  Returns (weights fp32 [T,k], ids int32 [T,k], token_expert_indices int32 [T,k] = j*T + t)."""
    x = gating.float()
    e = torch.exp(x - x.amax(dim=-1, keepdim=True))
    p = e * (1.0 / e.sum(dim=-1, keepdim=True))
    vals, ids = stable_topk(p, k)
    if renormalize:
        tot = torch.zeros(vals.shape[:-1], dtype=torch.float32)
        for j in range(k):
            tot = tot + vals[..., j]
        vals = vals / torch.where(tot > 0, tot, torch.ones_like(tot)).unsqueeze(-1)
    n = x.shape[0]
    src = (torch.arange(k).unsqueeze(0) * n + torch.arange(n).unsqueeze(1)).to(torch.int32)
    return vals, ids.to(torch.int32), src


def softmax_topk_margin(gating: torch.Tensor, k: int) -> torch.Tensor:
    """float64 decision margins of the softmax top-k: gaps between consecutive sorted logits at
    ranks 0..k (k gaps per row).  A CUDA/CPU id mismatch is excusable only where a gap is within a
    few fp32 ulps."""
    srt = torch.sort(gating.double(), dim=-1, descending=True).values
    return (srt[..., :k] - srt[..., 1:k + 1]).abs()


def _butterfly_sum8(v: torch.Tensor, T: torch.dtype = torch.float32) -> torch.Tensor:
    """Sum of 8 values in the order of an xor-butterfly with offsets 4, 2, 1, every partial sum
    rounded to T (kernel/fused_moe_gate_deepseek.cuh:324-327)."""
    a = rt(v[..., 0:4] + v[..., 4:8], T)
    b = rt(a[..., 0:2] + a[..., 2:4], T)
    return rt(b[..., 0] + b[..., 1], T)


def _larger_type(t1: torch.dtype, t2: torch.dtype) -> torch.dtype:
    # kernel/fused_moe_gate_deepseek.cuh:15-18: sizeof(T1) >= sizeof(T2) ? T1 : T2
    return t1 if t1.itemsize >= t2.itemsize else t2


def _gate_scores(gating: torch.Tensor, bias: torch.Tensor):
    """score = T1(1 / (1 + exp(-float(x)))); biased = ST(score + ST(bias)), ST the larger of the logit
    and bias dtypes (kernel/fused_moe_gate_deepseek.cuh:131-139).  Both returned widened to fp32."""
    T1 = gating.dtype
    ST = _larger_type(T1, bias.dtype)
    x = gating.float()
    score = rt(1.0 / (1.0 + torch.exp(-x)), T1)
    biased = rt(score + rt(bias.float(), ST).unsqueeze(0), ST)
    return score, biased, T1, ST


def fused_moe_gate_deepseek(gating: torch.Tensor, bias: torch.Tensor, topk: int, renormalize: bool,
                            num_expert_group: int, topk_group: int, routed_scaling: float = 1.0,
                            ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """mcoplib.op.fused_moe_gate_deepseek (moegate_type 0),
    kernel/fused_moe_gate_deepseek.cuh:129-243 (selection) and :316-332 (weights).

    score and biased score as _gate_scores (all fp32 for fp32 logits); group score = ST(sum of the two
    largest biased scores of the group); the `topk_group` best groups are kept (ties to the lower
    group); the top-k experts of the kept groups by biased score, ties to the lower expert id, in
    descending order; weight = float(T1(score / T1-sum of the selected scores)) * routed_scaling.
    Returns (weights fp32 [T,k], ids int32 [T,k], group_mask int32 [T] with bit g set iff group g kept)."""
    n, E = gating.shape
    score, biased, T1, ST = _gate_scores(gating, bias)
    G = max(int(num_expert_group), 1)
    if G > 1:
        grp = biased.reshape(n, G, E // G)
        top2 = torch.sort(grp, dim=-1, descending=True).values[..., :2]
        gscore = rt(top2[..., 0] + top2[..., 1], ST)
        _, gidx = stable_topk(gscore, topk_group)
        gmask = torch.zeros(n, G, dtype=torch.bool)
        gmask.scatter_(1, gidx, True)
        emask = gmask.unsqueeze(-1).expand(n, G, E // G).reshape(n, E)
        masked = torch.where(emask, biased, torch.full_like(biased, -float("inf")))
    else:
        gmask = torch.ones(n, 1, dtype=torch.bool)
        masked = biased
    _, ids = stable_topk(masked, topk)
    w = torch.gather(score, 1, ids)
    if renormalize:
        if topk == 8:
            tot = _butterfly_sum8(w, T1)
        else:
            tot = torch.zeros(n)
            for j in range(topk):
                tot = rt(tot + w[:, j], T1)
        w = rt(w / tot.unsqueeze(-1), T1)
    w = w * routed_scaling
    bits = (gmask.to(torch.int64) << torch.arange(gmask.shape[1]).unsqueeze(0)).sum(dim=1)
    return w.float(), ids.to(torch.int32), bits.to(torch.int32)


def fused_moe_gate_deepseek_sglang(gating: torch.Tensor, bias: torch.Tensor, topk: int, renormalize: bool,
                                   num_expert_group: int, topk_group: int, routed_scaling_factor: Optional[float] = None,
                                   num_fused_shared_experts: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """mcoplib.op.fused_moe_gate_deepseek with moegate_type 1 (SGLANG), kernel/fused_moe_gate_deepseek.cuh:334-374;
    host side op/fused_moe_gate_deepseek.cu:88-101 (scale_factor = 1.0f / routed_scaling_factor).
    PARITY UNPINNED (the reference's test covers moegate_type 0 only).

    Selection as moegate_type 0 (the shared expert replaces the LAST selected slot, so topk - shared routed experts
    remain).  s = T(sigmoid) of the routed experts; tot = fp32 sum in the order of a 16-lane xor-butterfly.
    One fused shared expert: last slot id = E, value T(T(tot) * T(scale_factor)).  With renormalize EVERY slot
    (the shared one too) becomes T(T(value) / T(tot)); routed weights are never scaled.
    Returns (weights fp32 [T, topk], ids int32 [T, topk])."""
    n, E = gating.shape
    shared = int(num_fused_shared_experts or 0)
    assert shared in (0, 1)
    routed = topk - shared
    assert routed <= 8
    _, ids, _ = fused_moe_gate_deepseek(gating, bias, routed, False, num_expert_group, topk_group, 1.0)
    T = gating.dtype
    score = _gate_scores(gating, bias)[0]
    w = torch.gather(score, 1, ids.long())
    p = torch.zeros(n, 8)
    p[:, :routed] = w
    tot = _butterfly_sum8(p, torch.float32)
    if shared:
        sf = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(
            1.0 if routed_scaling_factor is None else routed_scaling_factor, dtype=torch.float32)
        ws = rt(rt(tot, T) * rt(sf, T), T)
        w = torch.cat([w, ws.unsqueeze(-1)], dim=1)
        ids = torch.cat([ids, torch.full((n, 1), E, dtype=torch.int32)], dim=1)
    if renormalize:
        w = rt(rt(w, T) / rt(tot, T).unsqueeze(-1), T)
    return w.float(), ids.to(torch.int32)


def fused_moe_gate_opt(gating: torch.Tensor, bias: torch.Tensor, topk: int, renormalize: bool, num_expert_group: int,
                       topk_group: int, num_fused_shared_experts: int = 0,
                       routed_scaling_factor: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """mcoplib.op.fused_moe_gate_opt, op/moe_fused_gate_opt.cu:9-92; selection kernel/fused_moe_gate.cuh:137-251
    (grouped) and :253-343 (one group), weights :346-420.  Pinned by biased_grouped_topk of
    unit_test/test_fused_moe_gate_opt.py:78-135 (row-sorted ids exact, row-sorted weights to 1e-3).

    Selection as fused_moe_gate_deepseek with logits and bias of one dtype T.  Weights: s = T(sigmoid) of the
    selected experts; tot = fp32 sum in xor-butterfly order; w = float(T(s / T(tot))) when renormalize, else s;
    no scaling.  One fused shared expert: topk - 1 routed experts, last slot id = E and weight =
    float(double(fp32 butterfly sum of the routed w) * (1 / routed_scaling_factor)) when renormalize, else 0.
    Returns (weights fp32 [T, topk], ids int32 [T, topk])."""
    n, E = gating.shape
    shared = int(num_fused_shared_experts or 0)
    assert shared in (0, 1)
    routed = topk - shared
    assert routed <= 8
    _, ids, _ = fused_moe_gate_deepseek(gating, bias.to(gating.dtype), routed, False, num_expert_group, topk_group, 1.0)
    T = gating.dtype
    score = _gate_scores(gating, bias.to(gating.dtype))[0]
    w = torch.gather(score, 1, ids.long())

    def bsum(v):  # 16-lane butterfly with zeros beyond `routed`, fp32
        p = torch.zeros(n, 8)
        p[:, :routed] = v
        return _butterfly_sum8(p, torch.float32)

    if renormalize:
        w = rt(w / rt(bsum(w), T).unsqueeze(-1), T)
    if shared:
        mul = 1.0 / float(routed_scaling_factor if routed_scaling_factor is not None else 1.0)
        ws = (bsum(w).double() * mul).float() if renormalize else torch.zeros(n)
        w = torch.cat([w, ws.unsqueeze(-1)], dim=1)
        ids = torch.cat([ids, torch.full((n, 1), E, dtype=torch.int32)], dim=1)
    return w.float(), ids.to(torch.int32)


def grouped_topk(scores: torch.Tensor, n_group: int, topk_group: int, topk: int, renormalize: bool,
                 routed_scaling_factor: float, bias: torch.Tensor, scoring_func: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """torch.ops._moe_C.grouped_topk, op/vllm/moe/grouped_topk_kernels.cu: scoring :560-583, group scores :585-628,
    group and expert choice :700-775, weights :783-820.  Pinned (sigmoid scoring, fp32) by biased_grouped_topk of
    unit_test/test_fused_moe_gate_deepseek.py:15-70, the same routing rule (row-sorted ids exact, weights to 1e-3).

    score = x (scoring_func 0) or T(0.5 * tanh(0.5 * float(x)) + 0.5) (1); biased = T(score + float(bias));
    group score = T(best + second best biased score), not finite -> -inf; the topk_group best groups (ties to the
    lower group); the top-k biased scores of the kept groups whose logit is finite (ties to the lower expert id,
    descending order); value = float(score) * (float(scaling) / (1e-20 + fp32 butterfly sum of the selected
    scores)) when renormalize, else float(score) * float(scaling).  A token whose topk_group-th group score is -inf
    gets ids 0..k-1 and values 1/k.  Returns (values fp32 [T,k], ids int32 [T,k])."""
    n, E = scores.shape
    T = scores.dtype
    x = scores.float()
    score = x if scoring_func == 0 else rt(0.5 * torch.tanh(0.5 * x) + 0.5, T)
    biased = rt(score + bias.float().unsqueeze(0), T)
    G = max(int(n_group), 1)
    fallback = torch.zeros(n, dtype=torch.bool)
    if G > 1:
        grp = biased.reshape(n, G, E // G)
        top2 = torch.sort(grp, dim=-1, descending=True).values[..., :2]
        gscore = rt(top2[..., 0] + top2[..., 1], T)
        gscore = torch.where(torch.isfinite(gscore), gscore, torch.full_like(gscore, -float("inf")))
        gval, gidx = stable_topk(gscore, topk_group)
        fallback = gval[:, -1] == -float("inf")
        gmask = torch.zeros(n, G, dtype=torch.bool)
        gmask.scatter_(1, gidx, True)
        emask = gmask.unsqueeze(-1).expand(n, G, E // G).reshape(n, E)
        masked = torch.where(emask, biased, torch.full_like(biased, -float("inf")))
    else:
        masked = biased
    masked = torch.where(torch.isfinite(x), masked, torch.full_like(masked, -float("inf")))
    _, ids = stable_topk(masked, topk)
    w = torch.gather(score, 1, ids)
    scale = torch.full((n,), float(torch.tensor(routed_scaling_factor, dtype=torch.float32)))
    if renormalize:
        p = torch.zeros(n, 32)
        p[:, :topk] = w
        s = p
        for o in (16, 8, 4, 2, 1):  # xor butterfly over 32 lanes: lane i adds lane i ^ o
            s = s + s[:, torch.arange(32) ^ o]
        scale = scale / (torch.tensor(1e-20, dtype=torch.float32) + s[:, 0])
    w = w * scale.unsqueeze(-1)
    if bool(fallback.any()):
        w[fallback] = 1.0 / topk
        ids[fallback] = torch.arange(topk)
    return w.float(), ids.to(torch.int32)


def gate_margins(gating: torch.Tensor, bias: torch.Tensor, topk: int, num_expert_group: int,
                 topk_group: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """float64 margins of the grouped gate: (min gap between consecutive group scores around the
    kept/dropped boundary and inside the kept set is not needed for ids, so only the boundary gap is
    returned [T]; gaps between consecutive selected biased scores incl. the first dropped one [T,k])."""
    x = gating.double()
    n, E = x.shape
    biased = 1.0 / (1.0 + torch.exp(-x)) + bias.double().unsqueeze(0)
    G = max(int(num_expert_group), 1)
    if G > 1:
        grp = biased.reshape(n, G, E // G)
        top2 = torch.sort(grp, dim=-1, descending=True).values[..., :2]
        gs = torch.sort(top2.sum(-1), dim=-1, descending=True)
        gap_group = (gs.values[:, topk_group - 1] - gs.values[:, topk_group]).abs() if topk_group < G \
            else torch.full((n,), float("inf"), dtype=torch.float64)
        gmask = torch.zeros(n, G, dtype=torch.bool)
        gmask.scatter_(1, gs.indices[:, :topk_group], True)
        emask = gmask.unsqueeze(-1).expand(n, G, E // G).reshape(n, E)
        masked = torch.where(emask, biased, torch.full_like(biased, -float("inf")))
    else:
        gap_group = torch.full((n,), float("inf"), dtype=torch.float64)
        masked = biased
    srt = torch.sort(masked, dim=-1, descending=True).values
    return gap_group, (srt[:, :topk] - srt[:, 1:topk + 1]).abs()


def _scatter_order(ids: torch.Tensor, experts_per_rank: int):
    """Counting-sort order of the routing entries: (expert ascending, token ascending), ids outside
    [0, experts_per_rank) dropped (op/moe_scatter_dynamic_quant.cu:49-141,152-225).
    Returns (row2tok int32 [T*k] (-1 past the routed rows), counts, starts int32 [E], tok2row int32 [T,k] (-1 if dropped),
    order = flat (token, slot) index of every routed row)."""
    Tn, k = ids.shape
    R = Tn * k
    flat = ids.reshape(-1).long()
    tok = torch.arange(Tn).repeat_interleave(k)
    valid = (flat >= 0) & (flat < experts_per_rank)
    key = torch.where(valid, flat, torch.full_like(flat, experts_per_rank))
    order = torch.sort(key * Tn + tok, stable=True).indices
    nvalid = int(valid.sum())
    order = order[:nvalid]
    counts = torch.bincount(flat[valid], minlength=experts_per_rank).to(torch.int32)
    starts = (torch.cumsum(counts, 0) - counts).to(torch.int32)
    row2tok = torch.full((R,), -1, dtype=torch.int32)
    row2tok[:nvalid] = tok[order].to(torch.int32)
    tok2row = torch.full((Tn, k), -1, dtype=torch.int32)
    tok2row.reshape(-1)[order] = torch.arange(nvalid, dtype=torch.int32)
    return row2tok, counts, starts, tok2row, order


def moe_scatter_permutation(ids: torch.Tensor, experts_per_rank: int):
    """The index outputs of moe_scatter_dynamic_quant alone (no row arithmetic): (row2tok, counts, starts, tok2row)."""
    return _scatter_order(ids, experts_per_rank)[:4]


def moe_scatter_dynamic_quant(hidden: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                              smooth: torch.Tensor, experts_per_rank: int):
    """mcoplib.op.moe_scatter_dynamic_quant with no shared experts,
    op/moe_scatter_dynamic_quant.cu:49-141 (counts/starts), :152-225 (row order), :227-268 (row quant).
    PARITY UNPINNED (no reference test); the row arithmetic has the shape of
    smooth_per_token_dynamic_quant (unit_test/test_moe_swiglu_dq.py:6-14).

    Rows are ordered by (expert ascending, token ascending); ids outside [0, experts_per_rank) are
    dropped.  For row r of token t and expert e with j = first slot of t holding e:
    v = float(x[t]) * w[t,j] * smooth[e] (left to right, fp32); a = max|v|;
    scale[r] = float(double(a) * 0.0078740157); q = clamp(rne(v * (127 * (1/a))), -127, 127);
    an all-zero row yields codes 0 and scale 0.
    Returns (rows int8 [R,H], scales fp32 [R], row2tok int32 [R], counts int32 [E], starts int32 [E],
    tok2row int32 [T,k]); entries past the routed rows are 0 / -1."""
    Tn, H = hidden.shape
    k = ids.shape[1]
    R = Tn * k
    row2tok, counts, starts, tok2row, order = _scatter_order(ids, experts_per_rank)
    nvalid = order.numel()
    flat = ids.reshape(-1).long()
    tok = torch.arange(Tn).repeat_interleave(k)
    rows = torch.zeros(R, H, dtype=torch.int8)
    scales = torch.zeros(R, dtype=torch.float32)
    t_sel = tok[order]
    e_sel = flat[order]
    # weight of the FIRST slot of the token that holds this expert (lines 240-247)
    first_slot = (ids[t_sel].long() == e_sel.unsqueeze(1)).to(torch.int8).argmax(dim=1)
    w_sel = weights.float()[t_sel, first_slot]
    chunk = 4096
    for s0 in range(0, nvalid, chunk):
        sl = slice(s0, min(s0 + chunk, nvalid))
        v = hidden[t_sel[sl]].float() * w_sel[sl].unsqueeze(1) * smooth.float()[e_sel[sl]]
        a = v.abs().amax(dim=1)
        scales[sl] = (a.double() * 0.0078740157).float()
        sc = 127.0 * (1.0 / a)
        rows[sl] = float_to_int8_sym(v * sc.unsqueeze(1))
    return rows, scales, row2tok, counts, starts, tok2row


def moe_swiglu_dynamic_quantize(x: torch.Tensor, smooth: torch.Tensor, starts: torch.Tensor, counts: torch.Tensor,
                                experts: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """mcoplib.op.moe_swiglu_dynamic_quantize, op/moe_swiglu_dq.cu:63-118; the reference's own torch reference is
    moe_swiglu_dynamic_quant_run (unit_test/test_moe_swiglu_dq.py:16-44, silu(x1) * x2 then
    smooth_per_token_dynamic_quant per expert), which pins this function (codes atol 1).

    x [rows, 2H] = gate || up; rows of expert e are [starts[e], starts[e]+counts[e]);
    v = up * (gate * (1 / (1 + exp(-gate)))) * smooth[e] (fp32, left to right); a = max|v|;
    scale = float(double(a) * 0.0078740157); q = clamp(rne(v * (127 * (1/a))), -127, 127); a == 0 -> codes 0.
    Rows owned by no expert stay 0.  Returns (codes int8 [rows, H], scales fp32 [rows])."""
    rows, h2 = x.shape
    H = h2 // 2
    q = torch.zeros(rows, H, dtype=torch.int8)
    sc = torch.zeros(rows, dtype=torch.float32)
    for e in range(experts):
        a0, n = int(starts[e]), int(counts[e])
        if n <= 0:
            continue
        g = x[a0:a0 + n, :H].float()
        u = x[a0:a0 + n, H:].float()
        sig = g * (1.0 / (1.0 + torch.exp(-g)))
        v = u * sig * smooth[e].float().unsqueeze(0)
        a = v.abs().amax(dim=1)
        sc[a0:a0 + n] = (a.double() * 0.0078740157).float()
        mul = torch.where(a > 0, 127.0 * (1.0 / a), torch.zeros_like(a))
        q[a0:a0 + n] = float_to_int8_sym(v * mul.unsqueeze(1))
    return q, sc


def absmax_row_quant(v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row int8 quantisation shared by the silu_and_mul_*quant kernels of op/int8_quant_kernels.cu
    (:934-953, :1398-1417): a = max|v|; scale = float(double(a) * 0.0078740157); q = rne(v * (127 * (1/a)))
    saturated to int8 (|v * 127/a| <= 127 up to rounding, so the clamp never acts); a == 0 -> codes 0, scale 0.
    Pinned (codes atol 1, scales allclose) by the reference tests' ref_dynamic_per_token_quant
    (unit_test/test_silu_mul_dq_reorder_mask.py:12-45)."""
    a = v.abs().amax(dim=-1)
    sc = (a.double() * 0.0078740157).float()
    mul = torch.where(a > 0, 127.0 * (1.0 / a), torch.zeros_like(a))
    return float_to_int8_sym(v * mul.unsqueeze(-1)), sc


def silu_mul(x: torch.Tensor) -> torch.Tensor:
    """x [..., 2N] = gate || up in bf16/f16 -> fp32 up * (gate * (1 / (1 + exp(-gate)))), the expression of
    op/int8_quant_kernels.cu:1383-1386 (no rounding to the activation type before the quantisation)."""
    n = x.shape[-1] // 2
    g = x[..., :n].float()
    u = x[..., n:].float()
    return u * (g * (1.0 / (1.0 + torch.exp(-g))))


def fused_silu_mul_dq_reorder_quant(x: torch.Tensor, reorder_topk_ids: Optional[torch.Tensor], start_expert_id: int,
                                    end_expert_id: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """mcoplib.op.fused_silu_mul_dq_reorder_quant, op/int8_quant_kernels.cu:1355-1417,1893-1940.
    x [R, 2N]; row r is processed iff start <= reorder_topk_ids[r] <= end (all rows when ids is None: the form of
    fused_silu_mul_dq_quant_interface, :1877-1891).  The w2_scale argument of the reference is never applied:
    both branches of the interface instantiate the kernel with HAS_SCALE = false (:1908-1935).
    Returns (codes int8 [R, N], scales fp32 [R], active bool [R]); inactive rows are 0 here, untouched on the GPU.
    PARITY UNPINNED beyond absmax_row_quant: the reference test only prints error figures."""
    R, n2 = x.shape
    active = torch.ones(R, dtype=torch.bool) if reorder_topk_ids is None else \
        (reorder_topk_ids.long() >= start_expert_id) & (reorder_topk_ids.long() <= end_expert_id)
    q, sc = absmax_row_quant(silu_mul(x))
    q = torch.where(active.unsqueeze(1), q, torch.zeros_like(q))
    sc = torch.where(active, sc, torch.zeros_like(sc))
    return q, sc, active


def silu_mul_pack_stride(two_n: int) -> int:
    """Row stride, in activation elements, of the packed output of fused_silu_mul_dq_mask_quant
    (op/int8_quant_kernels.cu:1861): N code bytes + 4 scale bytes, rounded up to 256 elements."""
    return ((two_n // 4 + 2) + 255) // 256 * 256


def fused_silu_mul_dq_mask_quant(x: torch.Tensor, mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """mcoplib.op.fused_silu_mul_dq_mask_quant, op/int8_quant_kernels.cu:881-955,1844-1875.
    x [G, M, 2N]; mask [G] = valid rows per group.  Output rows are byte records of out_stride * 2 bytes:
    bytes [0, N) int8 codes, bytes [N, N+4) the fp32 scale; only rows m < mask[g] are written.
    Returns (packed uint8 [G, M, stride_bytes] with unwritten bytes 0, written bool [G, M]).
    The reference test checks the packed scale only (unit_test/test_silu_mul_dq_mask.py:223-236, rtol 1e-4,
    atol 1e-3 against a bf16-rounded Triton product); codes are pinned through absmax_row_quant."""
    G, M, n2 = x.shape
    n = n2 // 2
    stride_bytes = silu_mul_pack_stride(n2) * x.element_size()
    q, sc = absmax_row_quant(silu_mul(x))
    m_idx = torch.arange(M).unsqueeze(0)
    written = m_idx < mask.long().clamp(0, M).unsqueeze(1)
    packed = torch.zeros(G, M, stride_bytes, dtype=torch.uint8)
    packed[:, :, :n] = q.view(torch.uint8)
    packed[:, :, n:n + 4] = sc.contiguous().view(torch.uint8).reshape(G, M, 4)
    packed = torch.where(written.unsqueeze(-1), packed, torch.zeros_like(packed))
    return packed, written


def moe_gather(y: torch.Tensor, row2tok: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """mcoplib.op.moe_gather, op/moe_gather.cu:30-62,137-150: out[row2tok[r]] += y[r].
    PARITY UNPINNED.  The reference accumulates with bf16 atomics in an unspecified order; this
    oracle (and the build) fixes the order: acc = float(out[t]); acc += float(y[r]) for the rows of t
    in ascending r; out[t] = T(acc).  Rows with an id outside [0, T) are skipped."""
    Tn = out.shape[0]
    acc = out.float().clone()
    r2t = row2tok.long()
    valid = (r2t >= 0) & (r2t < Tn)
    rows = torch.nonzero(valid).reshape(-1)
    toks = r2t[rows]
    order = torch.sort(toks * (row2tok.numel() + 1) + rows).indices
    rows, toks = rows[order], toks[order]
    # occurrence index of every row within its token
    first = torch.searchsorted(toks, toks, right=False)
    occ = torch.arange(rows.numel()) - first
    for j in range(int(occ.max()) + 1 if rows.numel() else 0):
        m = occ == j
        acc[toks[m]] = acc[toks[m]] + y[rows[m]].float()
    return acc.to(out.dtype)


def moe_gather_bf16_sequential(y: torch.Tensor, row2tok: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One legal execution order of the reference's bf16 atomics (ascending rows, a rounding after
    every add), op/moe_gather.cu:55-60.  Used only to bound how far the fixed-order fp32 form may be
    from what the reference can produce."""
    T = out.dtype
    acc = out.clone()
    for r in range(y.shape[0]):
        t = int(row2tok[r])
        if 0 <= t < out.shape[0]:
            acc[t] = (acc[t].float() + y[r].float()).to(T)
    return acc


def moe_gather_weighted(y: torch.Tensor, row2tok: torch.Tensor, topk_ids: torch.Tensor,
                        topk_weights: torch.Tensor, starts: torch.Tensor, out: torch.Tensor,
                        accumulate: bool) -> torch.Tensor:
    """Weighted combine (no reference operator; weight lookup as op/moe_scatter_dynamic_quant.cu:240-247):
    expert of row r = the last e with starts[e] <= r (rows of an expert are contiguous), j = first slot
    of token t holding that expert; acc = float(out[t]) if accumulate else 0;
    acc = acc + fl(w[t,j] * float(y[r])) for the rows of t in ascending r (product and sum rounded
    separately in fp32); out[t] = T(acc)."""
    Tn = out.shape[0]
    R = row2tok.numel()
    acc = out.float().clone() if accumulate else torch.zeros(out.shape, dtype=torch.float32)
    r2t = row2tok.long()
    valid = (r2t >= 0) & (r2t < Tn)
    rows = torch.nonzero(valid).reshape(-1)
    toks = r2t[rows]
    exp = torch.searchsorted(starts.long().contiguous(), rows, right=True) - 1
    slot = (topk_ids[toks].long() == exp.unsqueeze(1)).to(torch.int8).argmax(dim=1)
    w = topk_weights.float()[toks, slot]
    order = torch.sort(toks * (R + 1) + rows).indices
    rows, toks, w = rows[order], toks[order], w[order]
    first = torch.searchsorted(toks, toks, right=False)
    occ = torch.arange(rows.numel()) - first
    for j in range(int(occ.max()) + 1 if rows.numel() else 0):
        m = occ == j
        acc[toks[m]] = acc[toks[m]] + w[m].unsqueeze(1) * y[rows[m]].float()
    return acc.to(out.dtype)


def moe_sum(inp: torch.Tensor) -> torch.Tensor:
    """torch.ops._moe_C.moe_sum, op/vllm/moe/moe_align_sum_kernels.cu:352-367 (kernel) and :770-815 (dispatch).

    inp [T, k, H] -> [T, H].  k in {2, 3, 4}: `scalar_t x = 0; x += in[k]` - the running sum lives in the
    element type, so every partial sum is rounded to it (0 + in[0] is exact).  Any other k: the reference calls
    at::sum_out, i.e. fp32 accumulation and one rounding; the order of that reduction is the framework's, the
    restatement adds the slots in order."""
    T, k, H = inp.shape
    if 2 <= k <= 4:
        acc = inp[:, 0].clone()
        for j in range(1, k):
            acc = (acc.float() + inp[:, j].float()).to(inp.dtype)
        return acc
    acc = torch.zeros(T, H, dtype=torch.float32)
    for j in range(k):
        acc = acc + inp[:, j].float()
    return acc.to(inp.dtype)


def moe_sum_reduce(inp: torch.Tensor, routed_scaling_factor: float) -> torch.Tensor:
    """sglang moe_sum_reduce, op/sglang/csrc/moe/moe_sum_reduce.cu:119-223: acc = 0 (fp32); acc += float(in[k]) in slot
    order; acc *= float(factor); one rounding to the element type.  The reference's own check
    (unit_test/test_moe_sum_reduce_triton.py:77-88) is torch.sum(input, dim=1) * factor compared by cosine similarity."""
    T, k, H = inp.shape
    acc = torch.zeros(T, H, dtype=torch.float32)
    for j in range(k):
        acc = acc + inp[:, j].float()
    acc = acc * torch.tensor(routed_scaling_factor, dtype=torch.float32)
    return acc.to(inp.dtype)


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int, max_num_tokens_padded: int,
                         expert_map: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """torch.ops._moe_C.moe_align_block_size, op/vllm/moe/moe_align_sum_kernels.cu:86-180 (counting, padded prefix,
    expert_ids, tail fill with 0) and :306-337 (placement).  Pinned by the bincount construction of
    benchmark/runners/mcoplib_mxbenchmark_moe_align_block_size_runners.py:62-80, which sorts every expert's range
    before comparing because the reference's placement order depends on its atomics; this restatement emits the
    ascending order directly.  (That runner pre-fills its expected expert_ids with -1; the kernel writes 0 to the
    blocks after the padded total, lines 174-179, and so does this function.)

    Returns (sorted_token_ids int32 [max_num_tokens_padded], expert_ids int32 [ceil(max/block)], total int32 [1])."""
    flat = topk_ids.reshape(-1).long()
    numel = flat.numel()
    e = flat.clone()
    valid = (e >= 0) & (e < num_experts)
    if expert_map is not None:
        m = expert_map.long()
        e = torch.where(valid, m[e.clamp(0, num_experts - 1)], torch.full_like(e, -1))
        valid = valid & (e >= 0) & (e < num_experts)
    sorted_ids = torch.full((max_num_tokens_padded,), numel, dtype=torch.int32)
    nblocks = (max_num_tokens_padded + block_size - 1) // block_size
    expert_ids = torch.zeros(nblocks, dtype=torch.int32)
    off = 0
    for ex in range(num_experts):
        idx = torch.nonzero(valid & (e == ex), as_tuple=True)[0]
        cnt = idx.numel()
        padded = (cnt + block_size - 1) // block_size * block_size
        hi = min(off + cnt, max_num_tokens_padded)
        if hi > off:
            sorted_ids[off:hi] = idx[:hi - off].to(torch.int32)
        b0, b1 = off // block_size, min((off + padded) // block_size, nblocks)
        if b1 > b0:
            expert_ids[b0:b1] = ex
        off += padded
    return sorted_ids, expert_ids, torch.tensor([off], dtype=torch.int32)
