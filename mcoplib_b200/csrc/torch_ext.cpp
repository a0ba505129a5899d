// Host shims: the operator surface of mcoplib for the hot path, over the mcop_b200 C ABI.
//
// Two surfaces are reproduced with the reference's argument order, in-place conventions and checks:
//   * the pybind11 module `op`  (mcoplib.op, op/pybind.cpp:30-104 of MetaX-MACA/mcoplib);
//   * torch library operators   (torch.ops._C.* and torch.ops._C_cache_ops.*, op/vllm/torch_bindings.cpp),
//     registered under the namespaces MCOP_TORCH_NS / MCOP_TORCH_NS_cache_ops (default mcop_C) because the
//     name `_C` is taken by any vLLM wheel present in the same process.
// Every function validates its tensors (TORCH_CHECK -> RuntimeError before any launch), takes the current
// CUDA stream and calls one extern "C" entry point.  No computation happens on the host and there is no
// fallback: without a CUDA device these functions raise.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <optional>
#include <string>
#include <tuple>

#include "mcop_b200.h"
#include "debug_trace.hpp"

#ifndef MCOP_TORCH_NS
#define MCOP_TORCH_NS mcop_C
#endif
#define MCOP_CAT_(a, b) a##b
#define MCOP_CAT(a, b) MCOP_CAT_(a, b)
#define MCOP_TORCH_NS_CACHE MCOP_CAT(MCOP_TORCH_NS, _cache_ops)
// the MoE routing operators of vLLM live in their own library: _moe_C beside _C, mcop_moe_C beside mcop_C
// (the build passes -DMCOP_TORCH_NS_MOE next to -DMCOP_TORCH_NS)
#ifndef MCOP_TORCH_NS_MOE
#define MCOP_TORCH_NS_MOE mcop_moe_C
#endif

namespace {

using at::Tensor;

int dtype_code(const Tensor& t, const char* what) {
  switch (t.scalar_type()) {
    case at::kFloat: return MCOP_F32;
    case at::kBFloat16: return MCOP_BF16;
    case at::kHalf: return MCOP_F16;
    default: TORCH_CHECK(false, what, ": unsupported dtype ", t.scalar_type());
  }
}

void check_rc(int rc) { TORCH_CHECK(rc == MCOP_OK, "mcop_b200: ", mcop_last_error()); }

void check_cuda(const Tensor& t, const char* name) { TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor"); }

mcop_stream_t cur_stream() { return reinterpret_cast<mcop_stream_t>(at::cuda::getCurrentCUDAStream().stream()); }

Tensor scratch_bytes(size_t bytes, const Tensor& like) {
  return at::empty({(int64_t)((bytes + 15) / 16 * 16)}, like.options().dtype(at::kByte));
}

// ---------------------------------------------------------------- part 1

// torch.ops._C.fused_add_rms_norm (op/vllm/layernorm_kernels.cu:243-292)
void fused_add_rms_norm(Tensor& input, Tensor& residual, Tensor& weight, double epsilon) {
  MCOP_DEBUG_CALL("fused_add_rms_norm", input, residual, weight, epsilon);
  check_cuda(input, "input");
  TORCH_CHECK(weight.scalar_type() == input.scalar_type());
  TORCH_CHECK(input.scalar_type() == residual.scalar_type());
  TORCH_CHECK(residual.is_contiguous());
  TORCH_CHECK(weight.is_contiguous());
  const int64_t hidden = input.size(-1);
  TORCH_CHECK(input.stride(-1) == 1 && input.dim() >= 1);
  const int64_t tokens = hidden ? input.numel() / hidden : 0;
  int64_t stride = hidden;
  if (input.dim() >= 2) {
    stride = input.stride(-2);
    // leading dims must collapse onto one row stride
    Tensor v = input.dim() > 2 ? input.view({-1, hidden}) : input;
    stride = v.stride(0);
  }
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_fused_add_rmsnorm(input.data_ptr(), stride, residual.data_ptr(), weight.data_ptr(), tokens, hidden,
                                  (float)epsilon, dtype_code(input, "fused_add_rms_norm"), cur_stream()));
}

// torch.ops._C.rms_norm_dynamic_per_token_quant
// (op/vllm/quantization/fused_kernels/fused_layernorm_dynamic_per_token_quant.cu:163-192) and
// mcoplib.op.rms_norm_dynamic_per_token_quant_custom (op/rms_norm_dynamic_per_token_quant.cu:266-285)
void rms_norm_dynamic_per_token_quant_vllm(Tensor& out, const Tensor& input, const Tensor& weight, Tensor& scales,
                                           double var_epsilon, std::optional<Tensor> scale_ub,
                                           std::optional<Tensor> residual) {
  MCOP_DEBUG_CALL("rms_norm_dynamic_per_token_quant_custom", out, input, weight, scales, var_epsilon, scale_ub, residual);
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == at::kChar, "only int8 output is built");
  TORCH_CHECK(out.is_contiguous() && input.is_contiguous());
  TORCH_CHECK(weight.scalar_type() == input.scalar_type());
  TORCH_CHECK(scales.scalar_type() == at::kFloat);
  if (scale_ub.has_value()) TORCH_CHECK(scale_ub->scalar_type() == at::kFloat);
  if (residual.has_value()) TORCH_CHECK(residual->scalar_type() == input.scalar_type() && residual->is_contiguous());
  const int64_t hidden = input.size(-1);
  const int64_t tokens = hidden ? input.numel() / hidden : 0;
  TORCH_CHECK(scales.numel() >= tokens && scales.is_contiguous(), "scales must hold one fp32 per token");
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_add_rmsnorm_quant_i8(out.data_ptr<int8_t>(), scales.data_ptr<float>(), input.data_ptr(), hidden,
                                     weight.data_ptr(), residual.has_value() ? residual->data_ptr() : nullptr,
                                     scale_ub.has_value() ? scale_ub->data_ptr<float>() : nullptr, tokens, hidden,
                                     (float)var_epsilon, dtype_code(input, "rms_norm_dynamic_per_token_quant"), cur_stream()));
}

// torch.ops._C.rms_norm_dynamic_per_token_quant: the reference allows scale_ub only with the fp8 output
// (fused_layernorm_dynamic_per_token_quant.cu:178-180: `if (scale_ub.has_value()) TORCH_CHECK(out.dtype() == kFp8Type)`);
// this build's output is int8, so the vLLM flavour refuses a bound while the `_custom` operator keeps honouring it.
void rms_norm_dynamic_per_token_quant_C(Tensor& out, const Tensor& input, const Tensor& weight, Tensor& scales, double var_epsilon,
                                        std::optional<Tensor> scale_ub, std::optional<Tensor> residual) {
  TORCH_CHECK(!(scale_ub.has_value() && out.scalar_type() == at::kChar),
              "rms_norm_dynamic_per_token_quant: scale_ub goes with the fp8 output only (the reference's rule); "
              "the int8 output takes no upper bound");
  rms_norm_dynamic_per_token_quant_vllm(out, input, weight, scales, var_epsilon, scale_ub, residual);
}

// sglang's rms_norm_dynamic_per_token_quant_custom with the extra normalised output
// (op/sglang/include/sgl_kernel_ops.h:138-145, op/sglang/csrc/elementwise/fused_layernorm_dynamic_per_token_quant_custom.cu:434-460)
void rms_norm_dynamic_per_token_quant_sgl(Tensor& out, Tensor& out_bf16, const Tensor& input, const Tensor& weight, Tensor& scales,
                                          double var_epsilon, std::optional<Tensor> scale_ub, std::optional<Tensor> residual) {
  MCOP_DEBUG_CALL("rms_norm_dynamic_per_token_quant_custom", out, out_bf16, input, weight, scales, var_epsilon, scale_ub, residual);
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == at::kChar, "only int8 output is built");
  TORCH_CHECK(out.is_contiguous() && input.is_contiguous());
  TORCH_CHECK(!scale_ub.has_value(), "scale_ub goes with the fp8 output only");  // the reference's rule (:451-453)
  TORCH_CHECK(scales.dtype() == torch::kFloat32);
  TORCH_CHECK(weight.scalar_type() == input.scalar_type() && out_bf16.scalar_type() == input.scalar_type() && out_bf16.is_contiguous() &&
              out_bf16.numel() == input.numel());
  if (residual.has_value()) TORCH_CHECK(residual->scalar_type() == input.scalar_type() && residual->is_contiguous());
  const int64_t hidden = input.size(-1);
  const int64_t tokens = hidden ? input.numel() / hidden : 0;
  TORCH_CHECK(scales.numel() >= tokens && scales.is_contiguous(), "scales must hold one fp32 per token");
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_add_rmsnorm_quant_i8_norm_out(out.data_ptr<int8_t>(), out_bf16.data_ptr(), scales.data_ptr<float>(), input.data_ptr(), hidden,
                                              weight.data_ptr(), residual.has_value() ? residual->data_ptr() : nullptr, nullptr, tokens,
                                              hidden, (float)var_epsilon, dtype_code(input, "rms_norm_dynamic_per_token_quant_custom"),
                                              cur_stream()));
}

// mcoplib.op.rms_norm_dynamic_per_token_quant, 9 arguments (op/fused_rms_norm_dq.cu:646-667)
void rms_norm_dynamic_per_token_quant_9(Tensor& out, const Tensor& input, const Tensor& weight, const Tensor& smooth_scale,
                                        Tensor& scales, double var_epsilon, Tensor& after_res, Tensor& after_norm,
                                        std::optional<Tensor> residual) {
  MCOP_DEBUG_CALL("rms_norm_dynamic_per_token_quant", out, input, weight, smooth_scale, scales, var_epsilon, after_res, after_norm, residual);
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == at::kChar);
  TORCH_CHECK(out.is_contiguous() && input.is_contiguous());
  TORCH_CHECK(scales.scalar_type() == at::kFloat);
  TORCH_CHECK(weight.scalar_type() == smooth_scale.scalar_type(), "weight and smooth_scale must share a dtype");
  TORCH_CHECK(weight.scalar_type() == at::kBFloat16 || weight.scalar_type() == at::kFloat, "weight must be bf16 or fp32");
  TORCH_CHECK(after_res.is_contiguous() && after_norm.is_contiguous() && weight.is_contiguous() && smooth_scale.is_contiguous());
  TORCH_CHECK(after_res.scalar_type() == input.scalar_type() && after_norm.scalar_type() == input.scalar_type());
  if (residual.has_value()) TORCH_CHECK(residual->scalar_type() == input.scalar_type() && residual->is_contiguous());
  const int64_t hidden = input.size(-1);
  const int64_t tokens = hidden ? input.numel() / hidden : 0;
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_rmsnorm_smooth_quant_i8(out.data_ptr<int8_t>(), scales.data_ptr<float>(), after_res.data_ptr(),
                                        after_norm.data_ptr(), input.data_ptr(), weight.data_ptr(), smooth_scale.data_ptr(),
                                        residual.has_value() ? residual->data_ptr() : nullptr, tokens, hidden,
                                        (float)var_epsilon, dtype_code(input, "rms_norm_dynamic_per_token_quant"),
                                        dtype_code(weight, "rms_norm_dynamic_per_token_quant weight"), cur_stream()));
}

// mcoplib.op.rms_norm (op/fused_rms_norm_dq.cu:980-999)
void rms_norm(Tensor& out, const Tensor& input, const Tensor& weight, double var_epsilon, std::optional<Tensor> after_res,
              std::optional<Tensor> residual, bool rms_div) {
  MCOP_DEBUG_CALL("rms_norm", out, input, weight, var_epsilon, after_res, residual, rms_div);
  check_cuda(input, "input");
  TORCH_CHECK(out.is_contiguous() && input.is_contiguous() && weight.is_contiguous());
  TORCH_CHECK(out.scalar_type() == input.scalar_type());
  TORCH_CHECK(after_res.has_value() == residual.has_value(), "after_res and residual go together");
  if (residual.has_value())
    TORCH_CHECK(residual->is_contiguous() && after_res->is_contiguous() && residual->scalar_type() == input.scalar_type() &&
                after_res->scalar_type() == input.scalar_type());
  const int64_t hidden = input.size(-1);
  const int64_t tokens = hidden ? input.numel() / hidden : 0;
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_rmsnorm(out.data_ptr(), input.data_ptr(), weight.data_ptr(), after_res.has_value() ? after_res->data_ptr() : nullptr,
                        residual.has_value() ? residual->data_ptr() : nullptr, tokens, hidden, (float)var_epsilon, rms_div ? 1 : 0,
                        dtype_code(input, "rms_norm"), dtype_code(weight, "rms_norm weight"), cur_stream()));
}

// mcoplib.op.head_rms_norm (op/fused_rms_norm_dq.cu:804-812)
void head_rms_norm(Tensor& out, const Tensor& hidden_states, const Tensor& weight, double var_epsilon, int head_offset, int head_norm) {
  MCOP_DEBUG_CALL("head_rms_norm", out, hidden_states, weight, var_epsilon, head_offset, head_norm);
  check_cuda(hidden_states, "hidden_states");
  TORCH_CHECK(hidden_states.dim() == 3, "hidden_states must be [tokens, heads, head_dim]");
  TORCH_CHECK(out.is_contiguous() && hidden_states.is_contiguous() && weight.is_contiguous());
  TORCH_CHECK(out.scalar_type() == hidden_states.scalar_type());
  const c10::cuda::OptionalCUDAGuard guard(device_of(hidden_states));
  check_rc(mcop_head_rmsnorm(out.data_ptr(), hidden_states.data_ptr(), weight.data_ptr(), hidden_states.size(0), hidden_states.size(1),
                             hidden_states.size(2), (float)var_epsilon, head_offset, head_norm, dtype_code(hidden_states, "head_rms_norm"),
                             dtype_code(weight, "head_rms_norm weight"), cur_stream()));
}

// mcoplib.op.scale_dynamic_quant (op/scale_dynamic_quant.cu:127-153): allocates and returns (codes, scales)
std::tuple<Tensor, Tensor> scale_dynamic_quant(const Tensor& hidden_states, const Tensor& smooth_scales, at::ScalarType dst) {
  MCOP_DEBUG_CALL("scale_dynamic_quant", hidden_states, smooth_scales, dst);
  check_cuda(hidden_states, "hidden_states");
  TORCH_CHECK(dst == at::kChar, "only int8 output is built");
  TORCH_CHECK(hidden_states.is_contiguous() && smooth_scales.is_contiguous());
  TORCH_CHECK(smooth_scales.scalar_type() == at::kFloat);
  const int64_t hidden = hidden_states.size(-1);
  const int64_t tokens = hidden ? hidden_states.numel() / hidden : 0;
  const c10::cuda::OptionalCUDAGuard guard(device_of(hidden_states));
  Tensor q = at::empty(hidden_states.sizes(), hidden_states.options().dtype(at::kChar));
  Tensor s = at::empty({tokens}, hidden_states.options().dtype(at::kFloat));
  check_rc(mcop_scale_dynamic_quant_i8(q.data_ptr<int8_t>(), s.data_ptr<float>(), hidden_states.data_ptr(), smooth_scales.data_ptr<float>(),
                                       tokens, hidden, dtype_code(hidden_states, "scale_dynamic_quant"), cur_stream()));
  return {q, s};
}

// torch.ops._C.dynamic_scaled_int8_quant (op/vllm/quantization/compressed_tensors/int8_quant_kernels.cu:459-526),
// symmetric form only (azp must be None)
void dynamic_scaled_int8_quant(Tensor& out, const Tensor& input, Tensor& scales, std::optional<Tensor> azp) {
  MCOP_DEBUG_CALL("dynamic_scaled_int8_quant", out, input, scales, azp);
  check_cuda(input, "input");
  TORCH_CHECK(input.is_contiguous());
  TORCH_CHECK(out.is_contiguous());
  TORCH_CHECK(scales.is_contiguous());
  TORCH_CHECK(!azp.has_value(), "asymmetric quantisation (azp) is not built");
  TORCH_CHECK(out.scalar_type() == at::kChar && scales.scalar_type() == at::kFloat);
  const int64_t hidden = input.size(-1);
  const int64_t tokens = hidden ? input.numel() / hidden : 0;
  TORCH_CHECK(scales.numel() >= tokens && out.numel() == input.numel());
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_dynamic_scaled_int8_quant(out.data_ptr<int8_t>(), scales.data_ptr<float>(), input.data_ptr(), tokens, hidden,
                                          dtype_code(input, "dynamic_scaled_int8_quant"), cur_stream()));
}

// ---------------------------------------------------------------- part 2

// torch.ops._C.rotary_embedding (op/vllm/pos_encoding_kernels.cu:135-217); the cos/sin cache may also be fp32
void rotary_embedding_vllm(Tensor& positions, Tensor& query, std::optional<Tensor> key, int64_t head_size, Tensor& cos_sin_cache,
                           bool is_neox) {
  MCOP_DEBUG_CALL("rotary_embedding", positions, query, key, head_size, cos_sin_cache, is_neox);
  check_cuda(query, "query");
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous());
  const int64_t num_tokens = positions.numel();
  const int positions_ndim = positions.dim();
  TORCH_CHECK(positions_ndim == 1 || positions_ndim == 2, "positions must have shape [num_tokens] or [batch_size, seq_len]");
  if (positions_ndim == 1) {
    TORCH_CHECK(query.size(0) == positions.size(0) && (!key.has_value() || key->size(0) == positions.size(0)),
                "query, key and positions must have the same number of tokens");
  } else {
    TORCH_CHECK(query.size(0) == positions.size(0) && (!key.has_value() || key->size(0) == positions.size(0)) &&
                    query.size(1) == positions.size(1) && (!key.has_value() || key->size(1) == positions.size(1)),
                "query, key and positions must have the same batch_size and seq_len");
  }
  const int64_t query_hidden = num_tokens ? query.numel() / num_tokens : 0;
  const int64_t key_hidden = key.has_value() && num_tokens ? key->numel() / num_tokens : 0;
  TORCH_CHECK(head_size > 0 && query_hidden % head_size == 0);
  TORCH_CHECK(key_hidden % head_size == 0);
  const int num_heads = (int)(query_hidden / head_size);
  const int num_kv_heads = key.has_value() ? (int)(key_hidden / head_size) : num_heads;
  TORCH_CHECK(num_kv_heads == 0 || num_heads % num_kv_heads == 0);
  TORCH_CHECK(cos_sin_cache.dim() == 2 && cos_sin_cache.size(0) > 0, "cos_sin_cache must be [max_position, rot_dim]");
  const int rot_dim = (int)cos_sin_cache.size(1);
  TORCH_CHECK(cos_sin_cache.is_contiguous());
  TORCH_CHECK(cos_sin_cache.scalar_type() == query.scalar_type() || cos_sin_cache.scalar_type() == at::kFloat,
              "cos_sin_cache must have the activation dtype or fp32");
  const int seq_dim_idx = positions_ndim - 1;
  const int64_t query_stride = query.stride(seq_dim_idx);
  const int64_t key_stride = key.has_value() ? key->stride(seq_dim_idx) : 0;
  const int query_ndim = query.dim();
  const int64_t head_stride = (query_ndim == positions_ndim + 2) ? query.stride(-2) : head_size;
  if (key.has_value()) TORCH_CHECK(key->scalar_type() == query.scalar_type());
  const c10::cuda::OptionalCUDAGuard guard(device_of(query));
  check_rc(mcop_rope_inplace(positions.data_ptr<int64_t>(), query.data_ptr(), key.has_value() ? key->data_ptr() : nullptr,
                             cos_sin_cache.data_ptr(), dtype_code(cos_sin_cache, "cos_sin_cache"), cos_sin_cache.size(0), num_tokens,
                             num_heads, num_kv_heads, (int)head_size, rot_dim, query_stride, key_stride, head_stride,
                             is_neox ? 1 : 0, dtype_code(query, "rotary_embedding"), cur_stream()));
}

// mcoplib.op.rotary_embedding (op/rotary_embedding.cu:99-121)
void rotary_embedding_packed(Tensor packed_qkv, Tensor q_len, Tensor accum_q_lens, Tensor cache_lens, Tensor cos, Tensor sin,
                             Tensor output, int q_head_num, int kv_head_num, int rope_offset) {
  MCOP_DEBUG_CALL("rotary_embedding", packed_qkv, q_len, accum_q_lens, cache_lens, cos, sin, output, q_head_num, kv_head_num, rope_offset);
  (void)rope_offset;  // accepted and unused, as in the reference (op/rotary_embedding.cu:68-70)
  (void)q_len;
  check_cuda(packed_qkv, "packed_qkv");
  TORCH_CHECK(packed_qkv.scalar_type() == at::kBFloat16, "Only bfloat16 are supported");
  TORCH_CHECK(packed_qkv.dim() == 3 && packed_qkv.is_contiguous() && output.is_contiguous());
  TORCH_CHECK(output.scalar_type() == packed_qkv.scalar_type() && output.sizes() == packed_qkv.sizes());
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() && sin.is_contiguous());
  TORCH_CHECK(accum_q_lens.scalar_type() == at::kInt && cache_lens.scalar_type() == at::kInt);
  const int64_t tokens = packed_qkv.size(0);
  const int head_dim = (int)packed_qkv.size(2);
  TORCH_CHECK(packed_qkv.size(1) == q_head_num + 2 * kv_head_num, "head count mismatch");
  TORCH_CHECK(cos.size(-1) * 2 == head_dim && sin.size(-1) * 2 == head_dim, "cos/sin must be [max_pos, head_dim/2]");
  const int batch = (int)cache_lens.numel();
  TORCH_CHECK(accum_q_lens.numel() >= batch + 1, "accum_q_lens must hold batch+1 entries");
  const c10::cuda::OptionalCUDAGuard guard(device_of(packed_qkv));
  const int64_t max_position = std::min(cos.numel(), sin.numel()) / (head_dim / 2);  // table rows both tensors hold
  TORCH_CHECK(max_position > 0, "cos/sin tables are empty");
  check_rc(mcop_rope_packed(packed_qkv.data_ptr(), output.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), max_position,
                            accum_q_lens.data_ptr<int32_t>(), cache_lens.data_ptr<int32_t>(), batch, tokens, q_head_num, kv_head_num,
                            head_dim, MCOP_BF16, cur_stream()));
}

// mcoplib.op.fused_rope_fwd / fused_rope_bwd (op/fused_rope.cu:13-74, 77-138): same checks, the rotation or its transpose
using FusedRopeFn = int (*)(void*, const void*, const void*, int64_t, const int64_t*, int64_t, int, int, int, int, int, mcop_stream_t);
static Tensor fused_rope_planes(const char* name, FusedRopeFn fn, Tensor qkv, const Tensor& cos, const Tensor& sin,
                                const std::optional<Tensor>& indexes, bool force_bf16_attn) {
  check_cuda(qkv, "qkv"); check_cuda(cos, "cos"); check_cuda(sin, "sin");
  TORCH_CHECK(qkv.is_contiguous() && cos.is_contiguous() && sin.is_contiguous());
  if (indexes.has_value()) {
    check_cuda(*indexes, "indexes");
    TORCH_CHECK(indexes->is_contiguous() && indexes->scalar_type() == at::kLong);
  }
  TORCH_CHECK(qkv.dim() == 4, "qkv must be [seq, 3, heads, head_dim]");
  TORCH_CHECK(qkv.scalar_type() == at::kHalf || qkv.scalar_type() == at::kBFloat16, "Only float16 and bfloat16 are supported");
  TORCH_CHECK(cos.scalar_type() == qkv.scalar_type() && sin.scalar_type() == qkv.scalar_type());
  TORCH_CHECK(cos.size(-1) * 2 == qkv.size(3));
  const c10::cuda::OptionalCUDAGuard guard(device_of(qkv));
  const int64_t max_position = std::min(cos.numel(), sin.numel()) / cos.size(-1);
  TORCH_CHECK(max_position > 0, "cos/sin tables are empty");
  const bool to_bf16 = force_bf16_attn && qkv.scalar_type() == at::kHalf;  // with bf16 data the flag changes nothing (op/fused_rope.cu:44-60)
  if (indexes.has_value()) TORCH_CHECK(indexes->numel() >= qkv.size(0), "indexes must hold one row number per sequence position");
  check_rc(fn(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), max_position, indexes.has_value() ? indexes->data_ptr<int64_t>() : nullptr,
              qkv.size(0), (int)qkv.size(1), (int)qkv.size(2), (int)qkv.size(3), dtype_code(qkv, name), to_bf16 ? 1 : 0, cur_stream()));
  // as the reference: the same storage, now holding bf16 in its Q and K planes, returned as a bf16 view
  return to_bf16 ? qkv.view(at::kBFloat16) : qkv;
}
Tensor fused_rope_fwd(Tensor qkv, Tensor cos, Tensor sin, std::optional<Tensor> indexes, bool force_bf16_attn) {
  MCOP_DEBUG_CALL("fused_rope_fwd", qkv, cos, sin, indexes, force_bf16_attn);
  return fused_rope_planes("fused_rope_fwd", &mcop_fused_rope_fwd, qkv, cos, sin, indexes, force_bf16_attn);
}
Tensor fused_rope_bwd(Tensor qkv, Tensor cos, Tensor sin, std::optional<Tensor> indexes, bool force_bf16_attn) {
  MCOP_DEBUG_CALL("fused_rope_bwd", qkv, cos, sin, indexes, force_bf16_attn);
  return fused_rope_planes("fused_rope_bwd", &mcop_fused_rope_bwd, qkv, cos, sin, indexes, force_bf16_attn);
}

// mcoplib.op.store_kv_cache_cuda_interface (op/store_kv.cu:220-350)
void store_kv_cache_cuda_interface(Tensor packed_qkv, Tensor q_lens, Tensor accum_q_lens, Tensor cache_lens, Tensor cache_slot_ids,
                                   Tensor& k_cache, Tensor& v_cache, Tensor k_scale, Tensor v_scale, int batch_size, int q_head_num,
                                   int kv_head_num) {
  MCOP_DEBUG_CALL("store_kv_cache_cuda_interface", packed_qkv, q_lens, accum_q_lens, cache_lens, cache_slot_ids, k_cache, v_cache, k_scale, v_scale, batch_size, q_head_num, kv_head_num);
  check_cuda(packed_qkv, "packed_qkv"); check_cuda(q_lens, "q_lens"); check_cuda(accum_q_lens, "accum_q_lens");
  check_cuda(cache_lens, "cache_lens"); check_cuda(cache_slot_ids, "cache_slot_ids"); check_cuda(k_cache, "k_cache");
  check_cuda(v_cache, "v_cache"); check_cuda(k_scale, "k_scale"); check_cuda(v_scale, "v_scale");
  TORCH_CHECK(packed_qkv.scalar_type() == at::kHalf || packed_qkv.scalar_type() == at::kBFloat16, "Only float16, bfloat16 are supported");
  TORCH_CHECK(packed_qkv.dim() == 3 && packed_qkv.stride(2) == 1);
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.dim() == 4 && k_cache.stride(3) == 1 && v_cache.stride(3) == 1);
  TORCH_CHECK(k_cache.size(1) >= kv_head_num && v_cache.size(1) >= kv_head_num && k_cache.size(3) >= packed_qkv.size(2) &&
                  v_cache.size(3) >= packed_qkv.size(2), "caches must be [slots, kv_heads, max_len, head_dim]");
  TORCH_CHECK(q_lens.numel() >= batch_size && accum_q_lens.numel() >= batch_size + 1 && cache_lens.numel() >= batch_size &&
                  cache_slot_ids.numel() >= batch_size && packed_qkv.size(1) >= q_head_num + 2 * kv_head_num,
              "length tensors must hold batch_size entries (accum_q_lens one more) and packed_qkv q + 2 kv heads");
  TORCH_CHECK(k_cache.scalar_type() == at::kChar && v_cache.scalar_type() == at::kChar);
  TORCH_CHECK(k_scale.scalar_type() == at::kFloat && v_scale.scalar_type() == at::kFloat && k_scale.is_contiguous() && v_scale.is_contiguous());
  TORCH_CHECK(q_lens.scalar_type() == at::kInt && accum_q_lens.scalar_type() == at::kInt && cache_lens.scalar_type() == at::kInt &&
              cache_slot_ids.scalar_type() == at::kInt);
  const int head_dim = (int)packed_qkv.size(2);
  TORCH_CHECK(k_scale.numel() == (int64_t)kv_head_num * head_dim && v_scale.numel() == (int64_t)kv_head_num * head_dim,
              "k_scale / v_scale must be [kv_heads, head_dim]");
  const c10::cuda::OptionalCUDAGuard guard(device_of(packed_qkv));
  check_rc(mcop_kv_store_i8(packed_qkv.data_ptr(), packed_qkv.stride(0), packed_qkv.stride(1), q_lens.data_ptr<int32_t>(),
                            accum_q_lens.data_ptr<int32_t>(), cache_lens.data_ptr<int32_t>(), cache_slot_ids.data_ptr<int32_t>(),
                            k_cache.data_ptr<int8_t>(), v_cache.data_ptr<int8_t>(), std::min(k_cache.size(0), v_cache.size(0)),
                            std::min(k_cache.size(2), v_cache.size(2)), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2),
                            v_cache.stride(0), v_cache.stride(1), v_cache.stride(2), k_scale.data_ptr<float>(), v_scale.data_ptr<float>(),
                            batch_size, packed_qkv.size(0), q_head_num, kv_head_num, head_dim, dtype_code(packed_qkv, "store_kv"), cur_stream()));
}

// torch.ops._C_cache_ops.reshape_and_cache_flash (op/vllm/cache_kernels.cu:610-650): only kv_cache_dtype "auto"
void reshape_and_cache_flash(Tensor& key, Tensor& value, Tensor& key_cache, Tensor& value_cache, Tensor& slot_mapping,
                             const std::string& kv_cache_dtype, Tensor& k_scale, Tensor& v_scale) {
  MCOP_DEBUG_CALL("reshape_and_cache_flash", key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale);
  (void)k_scale; (void)v_scale;
  check_cuda(key, "key");
  TORCH_CHECK(kv_cache_dtype == "auto", "only kv_cache_dtype \"auto\" is built (as in the reference)");
  TORCH_CHECK(key.dim() == 3 && value.dim() == 3 && key_cache.dim() == 4 && value_cache.dim() == 4);
  TORCH_CHECK(key_cache.scalar_type() == key.scalar_type() && value_cache.scalar_type() == value.scalar_type());
  TORCH_CHECK(slot_mapping.scalar_type() == at::kLong && slot_mapping.is_contiguous());
  TORCH_CHECK(key.stride(2) == 1 && value.stride(2) == 1 && key_cache.stride(3) == 1 && value_cache.stride(3) == 1);
  TORCH_CHECK(key.stride(1) == key.size(2) && value.stride(1) == value.size(2), "heads of key/value must be contiguous");
  TORCH_CHECK(key_cache.strides() == value_cache.strides(), "key_cache and value_cache must share a layout");
  const int64_t tokens = slot_mapping.size(0);
  const int kv_heads = (int)key.size(1), head_size = (int)key.size(2), block_size = (int)key_cache.size(1);
  TORCH_CHECK(key.size(0) >= tokens && value.size(0) >= tokens && value.size(1) == kv_heads && value.size(2) == head_size &&
                  key_cache.size(2) == kv_heads && key_cache.size(3) == head_size && key_cache.sizes() == value_cache.sizes(),
              "key/value must be [tokens, kv_heads, head_size] and the caches [num_blocks, block_size, kv_heads, head_size]");
  const c10::cuda::OptionalCUDAGuard guard(device_of(key));
  check_rc(mcop_reshape_and_cache_flash(key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0), key_cache.data_ptr(),
                                        value_cache.data_ptr(), key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
                                        slot_mapping.data_ptr<int64_t>(), tokens, kv_heads, head_size, block_size, key_cache.size(0),
                                        (int)key.element_size(), cur_stream()));
}

// torch.ops._C_cache_ops.reshape_and_cache (op/vllm/cache_kernels.cu:564-593): only kv_cache_dtype "auto";
// key_cache [num_blocks, kv_heads, head_size / x, block_size, x], value_cache [num_blocks, kv_heads, head_size, block_size]
void reshape_and_cache(Tensor& key, Tensor& value, Tensor& key_cache, Tensor& value_cache, Tensor& slot_mapping,
                       const std::string& kv_cache_dtype, Tensor& k_scale, Tensor& v_scale) {
  MCOP_DEBUG_CALL("reshape_and_cache", key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale);
  (void)k_scale; (void)v_scale;
  check_cuda(key, "key");
  TORCH_CHECK(kv_cache_dtype == "auto", "only kv_cache_dtype \"auto\" is built (as in the reference)");
  TORCH_CHECK(key.dim() == 3 && value.dim() == 3 && key_cache.dim() == 5 && value_cache.dim() == 4,
              "key/value must be [tokens, heads, head_size], key_cache [blocks, heads, head_size/x, block_size, x], "
              "value_cache [blocks, heads, head_size, block_size]");
  TORCH_CHECK(key_cache.scalar_type() == key.scalar_type() && value_cache.scalar_type() == value.scalar_type() &&
              key.scalar_type() == value.scalar_type());
  TORCH_CHECK(slot_mapping.scalar_type() == at::kLong && slot_mapping.is_contiguous());
  TORCH_CHECK(key_cache.is_contiguous() && value_cache.is_contiguous(), "the caches must be contiguous");
  TORCH_CHECK(key.stride(2) == 1 && value.stride(2) == 1 && key.stride(1) == key.size(2) && value.stride(1) == value.size(2),
              "heads of key/value must be contiguous");
  const int64_t tokens = slot_mapping.size(0);
  const int kv_heads = (int)key.size(1), head_size = (int)key.size(2);
  const int block_size = (int)key_cache.size(3), x = (int)key_cache.size(4);
  TORCH_CHECK(key.size(0) >= tokens && value.size(0) >= tokens && value.size(1) == kv_heads && value.size(2) == head_size);
  TORCH_CHECK(x > 0 && key_cache.size(1) == kv_heads && key_cache.size(2) * x == head_size && value_cache.size(0) == key_cache.size(0) &&
                  value_cache.size(1) == kv_heads && value_cache.size(2) == head_size && value_cache.size(3) == block_size,
              "cache shapes do not match key/value");
  const c10::cuda::OptionalCUDAGuard guard(device_of(key));
  check_rc(mcop_reshape_and_cache(key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0), key_cache.data_ptr(),
                                  value_cache.data_ptr(), slot_mapping.data_ptr<int64_t>(), tokens, kv_heads, head_size, block_size, x,
                                  key_cache.size(0), (int)key.element_size(), cur_stream()));
}

// Fused RoPE + int8 paged store (addition of this build, composition of the three ops above)
void rope_kv_store_int8(Tensor& positions, Tensor& query, Tensor& key, Tensor& value, int64_t head_size, Tensor& cos_sin_cache,
                        bool is_neox, Tensor& key_cache, Tensor& value_cache, Tensor& slot_mapping, Tensor& k_scale, Tensor& v_scale) {
  MCOP_DEBUG_CALL("rope_kv_store_int8", positions, query, key, value, head_size, cos_sin_cache, is_neox, key_cache, value_cache, slot_mapping, k_scale, v_scale);
  check_cuda(query, "query");
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous() && positions.dim() == 1);
  TORCH_CHECK(slot_mapping.scalar_type() == at::kLong && slot_mapping.is_contiguous());
  const int64_t tokens = positions.numel();
  TORCH_CHECK(query.dim() == 2 && key.dim() == 2 && value.dim() == 2, "query/key/value must be [tokens, heads*head_size]");
  TORCH_CHECK(query.size(0) == tokens && key.size(0) == tokens && value.size(0) == tokens && slot_mapping.numel() == tokens);
  TORCH_CHECK(query.stride(1) == 1 && key.stride(1) == 1 && value.stride(1) == 1);
  TORCH_CHECK(key.scalar_type() == query.scalar_type() && value.scalar_type() == query.scalar_type());
  TORCH_CHECK(head_size > 0 && query.size(1) % head_size == 0 && key.size(1) % head_size == 0 && value.size(1) == key.size(1));
  TORCH_CHECK(key_cache.scalar_type() == at::kChar && value_cache.scalar_type() == at::kChar);
  TORCH_CHECK(key_cache.dim() == 4 && key_cache.is_contiguous() && value_cache.is_contiguous() && key_cache.sizes() == value_cache.sizes(),
              "caches must be contiguous int8 [num_blocks, block_size, kv_heads, head_size]");
  const int num_heads = (int)(query.size(1) / head_size), num_kv_heads = (int)(key.size(1) / head_size);
  TORCH_CHECK(key_cache.size(2) == num_kv_heads && key_cache.size(3) == head_size);
  TORCH_CHECK(k_scale.scalar_type() == at::kFloat && v_scale.scalar_type() == at::kFloat && k_scale.numel() == num_kv_heads &&
              v_scale.numel() == num_kv_heads && k_scale.is_contiguous() && v_scale.is_contiguous());
  TORCH_CHECK(cos_sin_cache.is_contiguous() && cos_sin_cache.dim() == 2 && cos_sin_cache.size(0) > 0);
  const c10::cuda::OptionalCUDAGuard guard(device_of(query));
  check_rc(mcop_rope_kv_store_i8_paged(positions.data_ptr<int64_t>(), query.data_ptr(), key.data_ptr(), value.data_ptr(),
                                       cos_sin_cache.data_ptr(), dtype_code(cos_sin_cache, "cos_sin_cache"), cos_sin_cache.size(0),
                                       key_cache.data_ptr<int8_t>(),
                                       value_cache.data_ptr<int8_t>(), slot_mapping.data_ptr<int64_t>(), k_scale.data_ptr<float>(),
                                       v_scale.data_ptr<float>(), tokens, num_heads, num_kv_heads, (int)head_size, (int)cos_sin_cache.size(1),
                                       query.stride(0), key.stride(0), value.stride(0), (int)key_cache.size(1), key_cache.size(0),
                                       is_neox ? 1 : 0, dtype_code(query, "rope_kv_store_int8"), cur_stream()));
}

// ---------------------------------------------------------------- part 3

// mcoplib.op.moe_softmax_topk (op/moe_softmax_topk.cu:216-235)
void moe_softmax_topk(Tensor topk_weights, Tensor topk_indices, Tensor gating_output, bool pre_softmax) {
  MCOP_DEBUG_CALL("moe_softmax_topk", topk_weights, topk_indices, gating_output, pre_softmax);
  (void)pre_softmax;  // unused on this path in the reference as well: the weights are always renormalised
  check_cuda(gating_output, "gating_output");
  TORCH_CHECK(gating_output.scalar_type() == at::kFloat, "gating_output must be float32");
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat && topk_indices.scalar_type() == at::kInt);
  TORCH_CHECK(gating_output.is_contiguous() && topk_weights.is_contiguous() && topk_indices.is_contiguous());
  const int experts = (int)gating_output.size(-1);
  const int64_t tokens = experts ? gating_output.numel() / experts : 0;
  const int k = (int)topk_weights.size(-1);
  TORCH_CHECK(topk_weights.numel() == tokens * k && topk_indices.numel() == tokens * k);
  const c10::cuda::OptionalCUDAGuard guard(device_of(gating_output));
  check_rc(mcop_moe_softmax_topk(topk_weights.data_ptr<float>(), topk_indices.data_ptr<int32_t>(), gating_output.data_ptr<float>(), tokens,
                                 experts, k, cur_stream()));
}

// torch.ops._moe_C.topk_softmax (op/vllm/moe/topk_softmax_kernels.cu:884-918, schema op/vllm/moe/torch_bindings.cpp:6-9)
void topk_softmax(Tensor& topk_weights, Tensor& topk_indices, Tensor& token_expert_indices, Tensor& gating_output, bool renormalize) {
  MCOP_DEBUG_CALL("topk_softmax", topk_weights, topk_indices, token_expert_indices, gating_output, renormalize);
  check_cuda(gating_output, "gating_output");
  TORCH_CHECK(gating_output.scalar_type() == at::kFloat || gating_output.scalar_type() == at::kHalf ||
                  gating_output.scalar_type() == at::kBFloat16,
              "Unsupported gating_output data type: ", gating_output.scalar_type());
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat && topk_indices.scalar_type() == at::kInt &&
              token_expert_indices.scalar_type() == at::kInt);
  TORCH_CHECK(gating_output.is_contiguous() && topk_weights.is_contiguous() && topk_indices.is_contiguous() &&
              token_expert_indices.is_contiguous());
  const int experts = (int)gating_output.size(-1);
  const int64_t tokens = experts ? gating_output.numel() / experts : 0;
  const int k = (int)topk_weights.size(-1);
  TORCH_CHECK(topk_weights.numel() == tokens * k && topk_indices.numel() == tokens * k && token_expert_indices.numel() == tokens * k);
  const c10::cuda::OptionalCUDAGuard guard(device_of(gating_output));
  check_rc(mcop_topk_softmax(topk_weights.data_ptr<float>(), topk_indices.data_ptr<int32_t>(), token_expert_indices.data_ptr<int32_t>(),
                             gating_output.data_ptr(), tokens, experts, k, renormalize ? 1 : 0, dtype_code(gating_output, "topk_softmax"),
                             cur_stream()));
}

// torch.ops._moe_C.moe_sum (op/vllm/moe/moe_align_sum_kernels.cu:770-815): output [tokens, hidden] = sum over dim 1 of
// input [tokens, topk, hidden]
void moe_sum(Tensor& input, Tensor& output) {
  MCOP_DEBUG_CALL("moe_sum", input, output);
  check_cuda(input, "input"); check_cuda(output, "output");
  TORCH_CHECK(input.dim() == 3, "moe_sum: input must be [num_tokens, topk, hidden_size]");
  TORCH_CHECK(input.is_contiguous() && output.is_contiguous(), "moe_sum: tensors must be contiguous");
  TORCH_CHECK(input.scalar_type() == output.scalar_type(), "moe_sum: input and output dtypes differ");
  const int64_t hidden = input.size(-1);
  const int64_t tokens = hidden ? output.numel() / hidden : 0;
  TORCH_CHECK(tokens == input.size(0) && output.numel() == tokens * hidden, "moe_sum: output must be [num_tokens, hidden_size]");
  if (tokens == 0 || hidden == 0) return;
  const c10::cuda::OptionalCUDAGuard guard(device_of(output));
  check_rc(mcop_moe_sum(input.data_ptr(), output.data_ptr(), tokens, (int)input.size(1), hidden, dtype_code(input, "moe_sum"), cur_stream()));
}

// sglang's moe_sum_reduce (op/sglang/csrc/moe/moe_sum_reduce.cu:226-330): output = sum over dim 1 of input, times the factor
void moe_sum_reduce(Tensor& input, Tensor& output, double routed_scaling_factor) {
  MCOP_DEBUG_CALL("moe_sum_reduce", input, output, routed_scaling_factor);
  TORCH_CHECK(input.is_cuda(), "input must be CUDA tensor");
  TORCH_CHECK(output.is_cuda(), "output must be CUDA tensor");
  TORCH_CHECK(input.dim() == 3, "input must be a 3D tensor like [token_num, topk_num, hidden_dim]");
  TORCH_CHECK(output.dim() == 2, "output must be [token_num, hidden_dim]");
  TORCH_CHECK(input.size(0) == output.size(0), "token dim mismatch");
  TORCH_CHECK(input.size(2) == output.size(1), "hidden_dim mismatch");
  TORCH_CHECK(input.is_contiguous(), "expect input to be contiguous");
  TORCH_CHECK(output.is_contiguous(), "expect output to be contiguous");
  TORCH_CHECK(input.scalar_type() == output.scalar_type(), "moe_sum_reduce: input and output dtypes differ");
  if (input.size(0) == 0 || input.size(2) == 0) return;
  TORCH_CHECK(input.size(1) >= 1, "moe_sum_reduce: topk_num must be at least 1");
  const c10::cuda::OptionalCUDAGuard guard(device_of(output));
  check_rc(mcop_moe_sum_reduce(input.data_ptr(), output.data_ptr(), input.size(0), (int)input.size(1), input.size(2),
                               routed_scaling_factor, dtype_code(input, "moe_sum_reduce"), cur_stream()));
}

// torch.ops._moe_C.moe_align_block_size (op/vllm/moe/moe_align_sum_kernels.cu:612-735)
void moe_align_block_size(Tensor topk_ids, int64_t num_experts, int64_t block_size, Tensor sorted_token_ids, Tensor experts_ids,
                          Tensor num_tokens_post_pad, std::optional<Tensor> maybe_expert_map) {
  MCOP_DEBUG_CALL("moe_align_block_size", topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad,
                  maybe_expert_map);
  check_cuda(topk_ids, "topk_ids"); check_cuda(sorted_token_ids, "sorted_token_ids"); check_cuda(experts_ids, "experts_ids");
  check_cuda(num_tokens_post_pad, "num_tokens_post_pad");
  TORCH_CHECK(block_size > 0, "block_size should be greater than 0. ");
  TORCH_CHECK(num_experts > 0 && num_experts < 1024, "padded_num_experts must be less than 1024");
  TORCH_CHECK(c10::isIntegralType(topk_ids.scalar_type(), false), "moe_align_block_size: topk_ids must be an integer tensor");
  TORCH_CHECK(sorted_token_ids.scalar_type() == at::kInt && experts_ids.scalar_type() == at::kInt &&
              num_tokens_post_pad.scalar_type() == at::kInt, "moe_align_block_size: outputs must be int32");
  TORCH_CHECK(sorted_token_ids.is_contiguous() && experts_ids.is_contiguous() && num_tokens_post_pad.numel() >= 1);
  const c10::cuda::OptionalCUDAGuard guard(device_of(topk_ids));
  // the kernels read int32 ids; other integer types (the reference dispatches over all of them) are converted first
  const Tensor ids = topk_ids.scalar_type() == at::kInt && topk_ids.is_contiguous() ? topk_ids : topk_ids.to(at::kInt).contiguous();
  Tensor map;
  if (maybe_expert_map.has_value()) {
    check_cuda(*maybe_expert_map, "expert_map");
    TORCH_CHECK(maybe_expert_map->numel() >= num_experts, "moe_align_block_size: expert_map shorter than num_experts");
    map = maybe_expert_map->scalar_type() == at::kInt && maybe_expert_map->is_contiguous() ? *maybe_expert_map
                                                                                           : maybe_expert_map->to(at::kInt).contiguous();
  }
  const int64_t numel = ids.numel();
  const int64_t cap = sorted_token_ids.size(0);
  const int64_t blocks = std::min<int64_t>((cap + block_size - 1) / block_size, experts_ids.numel());
  const size_t ws_bytes = mcop_moe_align_block_size_workspace_bytes(numel, (int)num_experts);
  Tensor ws = scratch_bytes(ws_bytes, sorted_token_ids);
  check_rc(mcop_moe_align_block_size(numel ? ids.data_ptr<int32_t>() : nullptr, numel, (int)num_experts, (int)block_size,
                                     sorted_token_ids.data_ptr<int32_t>(), cap, experts_ids.data_ptr<int32_t>(), blocks,
                                     num_tokens_post_pad.data_ptr<int32_t>(), map.defined() ? map.data_ptr<int32_t>() : nullptr,
                                     ws.data_ptr(), ws_bytes, cur_stream()));
}

// sglang's store_kv_cache (op/sglang/csrc/memory/store.cu:72-150): k_cache[out_loc[i], :] = k[i, :], same for v; rows are
// the flattened trailing dimensions, a multiple of 128 bytes as in the reference
void store_kv_cache(Tensor k_cache, Tensor v_cache, Tensor out_loc, Tensor k, Tensor v) {
  MCOP_DEBUG_CALL("store_kv_cache", k_cache, v_cache, out_loc, k, v);
  const int64_t max_tokens = k_cache.size(0);
  const int64_t num_tokens = out_loc.size(0);
  k_cache = k_cache.view({max_tokens, -1});
  v_cache = v_cache.view({max_tokens, -1});
  k = k.view({num_tokens, -1});
  v = v.view({num_tokens, -1});
  TORCH_CHECK(k_cache.is_cuda() && v_cache.is_cuda() && out_loc.is_cuda() && k.is_cuda() && v.is_cuda(), "All tensors must be CUDA tensors");
  TORCH_CHECK(k_cache.sizes() == v_cache.sizes(), "k_cache and v_cache must have the same size");
  TORCH_CHECK(k_cache.strides() == v_cache.strides(), "k_cache and v_cache must have the same strides");
  TORCH_CHECK(k.sizes() == v.sizes(), "k and v must have the same size");
  TORCH_CHECK(k.strides() == v.strides(), "k and v must have the same strides");
  TORCH_CHECK(k.stride(-1) == 1 && k_cache.stride(-1) == 1, "k and k_cache must be contiguous in head.");
  TORCH_CHECK(k.size(-1) == k_cache.size(-1), "k and k_cache must have the same head size");
  TORCH_CHECK(out_loc.dim() == 1 && out_loc.is_contiguous(), "out_loc must be a 1D contiguous tensor");
  TORCH_CHECK(out_loc.scalar_type() == at::kInt || out_loc.scalar_type() == at::kLong, "out_loc must be of type int32 or int64, got: ",
              out_loc.scalar_type());
  TORCH_CHECK(k.scalar_type() == k_cache.scalar_type() && v.scalar_type() == v_cache.scalar_type());
  const int64_t size_bytes = k.element_size() * k.size(-1);
  TORCH_CHECK(size_bytes % 128 == 0, "The last dimension size bytes of k and v must be divisible by 128 at least, got: ", size_bytes);
  const c10::cuda::OptionalCUDAGuard guard(device_of(k));
  const Tensor loc = out_loc.scalar_type() == at::kLong ? out_loc : out_loc.to(at::kLong);
  check_rc(mcop_reshape_and_cache_flash(k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                                        k_cache.stride(0), 0, 0, loc.data_ptr<int64_t>(), num_tokens, 1, (int)k.size(-1), 1, max_tokens,
                                        (int)k.element_size(), cur_stream()));
}

// sglang's apply_rope_pos_ids_cos_sin_cache (op/sglang/csrc/elementwise/rope.cu:28-171): RoPE from an fp32 cos||sin cache at
// explicit positions, written to q_rope / k_rope (which may be q / k), optionally followed by
// k_buffer[kv_cache_loc[i]] = k_rope[i], v_buffer[kv_cache_loc[i]] = v[i].  fp32 products and sum, one rounding.
// With the save, NeoX order and rotary_dim == head_dim this is ONE call (mcop_rope_kv_copy); other forms rotate, then copy.
void apply_rope_pos_ids_cos_sin_cache(Tensor q, Tensor k, Tensor q_rope, Tensor k_rope, Tensor cos_sin_cache, Tensor pos_ids, bool interleave,
                                      bool enable_pdl, const std::optional<Tensor>& v, const std::optional<Tensor>& k_buffer,
                                      const std::optional<Tensor>& v_buffer, const std::optional<Tensor>& kv_cache_loc) {
  MCOP_DEBUG_CALL("apply_rope_pos_ids_cos_sin_cache", q, k, q_rope, k_rope, cos_sin_cache, pos_ids, interleave, enable_pdl, v, k_buffer,
                  v_buffer, kv_cache_loc);
  check_cuda(q, "q");
  const bool save_kv_cache = v.has_value();
  if (save_kv_cache) {
    TORCH_CHECK(k_buffer.has_value());
    TORCH_CHECK(v_buffer.has_value());
    TORCH_CHECK(kv_cache_loc.has_value());
    TORCH_CHECK(v->stride(-1) == 1 && k_buffer->stride(-1) == 1 && v_buffer->stride(-1) == 1);
    TORCH_CHECK(k_buffer->dim() == 3 && v_buffer->dim() == 3 && v->dim() == 3 && kv_cache_loc->dim() == 1);
    TORCH_CHECK(kv_cache_loc->is_cuda() && kv_cache_loc->is_contiguous() && kv_cache_loc->scalar_type() == at::kLong);
  } else {
    TORCH_CHECK(!enable_pdl);
  }
  TORCH_CHECK(q.stride(-1) == 1 && k.stride(-1) == 1 && q_rope.stride(-1) == 1 && k_rope.stride(-1) == 1);
  TORCH_CHECK(cos_sin_cache.is_cuda() && cos_sin_cache.is_contiguous() && pos_ids.is_cuda() && pos_ids.is_contiguous());
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && cos_sin_cache.dim() == 2);
  TORCH_CHECK(q.size(0) == k.size(0) && q.size(2) == k.size(2));
  TORCH_CHECK(cos_sin_cache.scalar_type() == at::kFloat && pos_ids.scalar_type() == at::kLong);
  TORCH_CHECK(q.scalar_type() == at::kHalf || q.scalar_type() == at::kBFloat16, "q must be fp16 or bf16");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && q_rope.scalar_type() == q.scalar_type() && k_rope.scalar_type() == q.scalar_type());
  TORCH_CHECK(q_rope.sizes() == q.sizes() && k_rope.sizes() == k.sizes());
  const int64_t nnz = q.size(0);
  const int heads = (int)q.size(1), kv_heads = (int)k.size(1), head_dim = (int)q.size(2), rot = (int)cos_sin_cache.size(1);
  const c10::cuda::OptionalCUDAGuard guard(device_of(q));
  // the rotation kernels work in place: a separate destination first receives a copy (this also carries the
  // non-rotated tail of every head when rotary_dim < head_dim)
  if (q_rope.data_ptr() != q.data_ptr()) q_rope.copy_(q);
  if (k_rope.data_ptr() != k.data_ptr()) k_rope.copy_(k);
  TORCH_CHECK(q_rope.stride(1) == k_rope.stride(1), "q_rope and k_rope must have one head stride");
  TORCH_CHECK(pos_ids.numel() >= nnz && cos_sin_cache.size(0) > 0);
  if (save_kv_cache && !interleave && rot == head_dim && q_rope.stride(1) == head_dim && k_rope.stride(1) == head_dim &&
      v->stride(1) == head_dim && k_buffer->stride(1) == head_dim && k_buffer->strides() == v_buffer->strides() &&
      k_buffer->size(1) == kv_heads && k_buffer->size(2) == head_dim && v->size(0) == nnz && v->size(1) == kv_heads &&
      v->size(2) == head_dim && kv_cache_loc->numel() == nnz && v->scalar_type() == q.scalar_type() &&
      k_buffer->scalar_type() == q.scalar_type() && v_buffer->scalar_type() == q.scalar_type()) {
    // rotation and save in one call (one launch from 2048 tokens on, like the reference's fused kernel)
    check_rc(mcop_rope_kv_copy(pos_ids.data_ptr<int64_t>(), q_rope.data_ptr(), k_rope.data_ptr(), v->data_ptr(),
                               cos_sin_cache.data_ptr<float>(), cos_sin_cache.size(0), k_buffer->data_ptr(), v_buffer->data_ptr(),
                               kv_cache_loc->data_ptr<int64_t>(), std::min(k_buffer->size(0), v_buffer->size(0)), k_buffer->stride(0), nnz,
                               heads, kv_heads, head_dim, q_rope.stride(0), k_rope.stride(0), v->stride(0),
                               dtype_code(q, "apply_rope_pos_ids_cos_sin_cache"), cur_stream()));
    return;
  }
  check_rc(mcop_rope_inplace(pos_ids.data_ptr<int64_t>(), q_rope.data_ptr(), k_rope.data_ptr(), cos_sin_cache.data_ptr(), MCOP_F32,
                             cos_sin_cache.size(0), nnz, heads,
                             kv_heads, head_dim, rot, q_rope.stride(0), k_rope.stride(0), q_rope.stride(1), interleave ? 0 : 1,
                             dtype_code(q, "apply_rope_pos_ids_cos_sin_cache"), cur_stream()));
  if (save_kv_cache) {
    TORCH_CHECK(v->scalar_type() == q.scalar_type() && k_buffer->scalar_type() == q.scalar_type() && v_buffer->scalar_type() == q.scalar_type());
    TORCH_CHECK(v->size(0) == nnz && v->size(1) == kv_heads && v->size(2) == head_dim && kv_cache_loc->numel() == nnz);
    TORCH_CHECK(k_rope.stride(1) == head_dim && v->stride(1) == head_dim, "heads of k_rope and v must be contiguous for the buffer save");
    TORCH_CHECK(k_buffer->strides() == v_buffer->strides() && k_buffer->size(1) == kv_heads && k_buffer->size(2) == head_dim,
                "k_buffer and v_buffer must share one [*, kv_heads, head_dim] layout");
    check_rc(mcop_reshape_and_cache_flash(k_rope.data_ptr(), v->data_ptr(), k_rope.stride(0), v->stride(0), k_buffer->data_ptr(),
                                          v_buffer->data_ptr(), k_buffer->stride(0), 0, k_buffer->stride(1),
                                          kv_cache_loc->data_ptr<int64_t>(), nnz, kv_heads, head_dim, 1,
                                          std::min(k_buffer->size(0), v_buffer->size(0)), (int)q.element_size(), cur_stream()));
  }
}

// torch.ops._moe_C.grouped_topk (op/vllm/moe/grouped_topk_kernels.cu:962-1060): allocates and returns (values, indices)
std::tuple<Tensor, Tensor> grouped_topk(const Tensor& scores, int64_t n_group, int64_t topk_group, int64_t topk, bool renormalize,
                                        double routed_scaling_factor, const Tensor& bias, int64_t scoring_func) {
  MCOP_DEBUG_CALL("grouped_topk", scores, n_group, topk_group, topk, renormalize, routed_scaling_factor, bias, scoring_func);
  check_cuda(scores, "scores");
  TORCH_CHECK(scores.dim() == 2, "scores must be a 2D Tensor");
  const int64_t tokens = scores.size(0), experts = scores.size(1);
  TORCH_CHECK(n_group >= 1 && experts % n_group == 0, "num_experts should be divisible by n_group");
  TORCH_CHECK(n_group <= 32, "n_group should be smaller than or equal to 32 for now");
  TORCH_CHECK(topk <= 32, "topk should be smaller than or equal to 32 for now");
  TORCH_CHECK(scoring_func == 0 || scoring_func == 1, "scoring_func must be SCORING_NONE (0) or SCORING_SIGMOID (1)");
  TORCH_CHECK(scores.is_contiguous() && bias.is_contiguous() && bias.numel() == experts);
  const c10::cuda::OptionalCUDAGuard guard(device_of(scores));
  Tensor values = at::empty({tokens, topk}, scores.options().dtype(at::kFloat));
  Tensor indices = at::empty({tokens, topk}, scores.options().dtype(at::kInt));
  check_rc(mcop_grouped_topk(scores.data_ptr(), bias.data_ptr(), values.data_ptr<float>(), indices.data_ptr<int32_t>(), tokens, (int)experts,
                             (int)n_group, (int)topk_group, (int)topk, renormalize ? 1 : 0, routed_scaling_factor, (int)scoring_func,
                             dtype_code(scores, "scores"), dtype_code(bias, "bias"), cur_stream()));
  return {values, indices};
}

// mcoplib.op.fused_moe_gate_deepseek (op/fused_moe_gate_deepseek.cu:63-138)
int fused_moe_gate_deepseek(Tensor& gating_outputs, Tensor& correction_bias, Tensor& out_routing_weights, Tensor& out_selected_experts,
                            int topk, bool renormalize, int num_expert_group, int topk_group,
                            std::optional<int> num_fused_shared_experts, std::optional<float> routed_scaling_factor,
                            std::optional<int> moegate_type, std::optional<Tensor> debug_group_mask) {
  MCOP_DEBUG_CALL("fused_moe_gate_deepseek", gating_outputs, correction_bias, out_routing_weights, out_selected_experts, topk, renormalize, num_expert_group, topk_group, num_fused_shared_experts, routed_scaling_factor, moegate_type, debug_group_mask);
  check_cuda(gating_outputs, "gating_outputs");
  TORCH_CHECK(gating_outputs.dim() == 2 && gating_outputs.is_contiguous() && correction_bias.is_contiguous());
  TORCH_CHECK(out_routing_weights.scalar_type() == at::kFloat && out_routing_weights.is_contiguous());
  TORCH_CHECK(out_selected_experts.scalar_type() == at::kInt && out_selected_experts.is_contiguous(), "selected experts must be int32");
  // the reference's argument checks, in its order (op/fused_moe_gate_deepseek.cu:77-101)
  const int moe_type = moegate_type.value_or(0);
  TORCH_CHECK(moe_type >= 0 && moe_type < 2, "Expected moegate_type == DEEPSEEK(0) or SGLANG(1), but get ", moe_type);
  // (the reference takes topk 8 or 9 only; every topk the kernel supports is accepted here)
  const int num_shared = num_fused_shared_experts.value_or(0);
  if (num_shared > 0) TORCH_CHECK(topk >= 9, "Expected topk >= 9 when fused_num_shared_experts > 0, but get topk = ", topk);
  TORCH_CHECK(num_shared == 0 || moe_type == 1, "Invalid arguments: fused shared experts go with moegate_type 1 only");
  TORCH_CHECK(num_shared <= 1, "more than one fused shared expert is not built (the reference draws their ids from the clock)");
  const int64_t tokens = gating_outputs.size(0);
  const int experts = (int)gating_outputs.size(1);
  TORCH_CHECK(correction_bias.numel() == experts);
  TORCH_CHECK(out_routing_weights.numel() == tokens * topk && out_selected_experts.numel() == tokens * topk);
  int32_t* gm = nullptr;
  if (debug_group_mask.has_value()) {
    TORCH_CHECK(debug_group_mask->scalar_type() == at::kInt && debug_group_mask->numel() == tokens && debug_group_mask->is_contiguous());
    gm = debug_group_mask->data_ptr<int32_t>();
  }
  const c10::cuda::OptionalCUDAGuard guard(device_of(gating_outputs));
  check_rc(mcop_moe_gate_grouped_sigmoid(gating_outputs.data_ptr(), correction_bias.data_ptr(), out_routing_weights.data_ptr<float>(),
                                         out_selected_experts.data_ptr<int32_t>(), gm, tokens, experts, num_expert_group, topk_group, topk,
                                         renormalize ? 1 : 0, routed_scaling_factor.value_or(1.0f), num_shared, moe_type,
                                         dtype_code(gating_outputs, "gating_outputs"), dtype_code(correction_bias, "correction_bias"),
                                         cur_stream()));
  return 0;
}

// mcoplib.op.fused_moe_gate_opt (op/moe_fused_gate_opt.cu:9-92): the reference's argument checks, in its order
int64_t fused_moe_gate_opt(Tensor& gating_outputs, Tensor& correction_bias, Tensor& out_routing_weights, Tensor& out_selected_experts,
                           int64_t topk, bool renormalize, int64_t num_expert_group, int64_t topk_group,
                           std::optional<int64_t> num_fused_shared_experts, std::optional<double> routed_scaling_factor) {
  MCOP_DEBUG_CALL("fused_moe_gate_opt", gating_outputs, correction_bias, out_routing_weights, out_selected_experts, topk, renormalize, num_expert_group, topk_group, num_fused_shared_experts, routed_scaling_factor);
  check_cuda(gating_outputs, "gating_outputs");
  TORCH_CHECK(((topk == 8) || (topk == 9)), "Expected topk = 8, but get topk = ", topk);
  const int64_t num_shared = num_fused_shared_experts.value_or(0);
  if (num_shared > 0) TORCH_CHECK(topk >= 9, "Expected topk >= 9 when fused_num_shared_experts > 0, but get topk = ", topk);
  if (num_shared == 0) TORCH_CHECK(topk == 8, "Expected topk == 8 when fused_num_shared_experts = 0 or None, but get topk = ", topk);
  TORCH_CHECK(num_shared <= 1, "more than one fused shared expert is not built (the reference draws their ids from rand())");
  TORCH_CHECK(gating_outputs.dim() == 2 && gating_outputs.is_contiguous() && correction_bias.is_contiguous());
  TORCH_CHECK(correction_bias.scalar_type() == gating_outputs.scalar_type(), "bias and logits must have one dtype");
  TORCH_CHECK(out_routing_weights.scalar_type() == at::kFloat && out_routing_weights.is_contiguous());
  TORCH_CHECK(out_selected_experts.scalar_type() == at::kInt && out_selected_experts.is_contiguous(), "selected experts must be int32");
  const int64_t tokens = gating_outputs.size(0);
  const int64_t experts = gating_outputs.size(1);
  const bool known = (num_expert_group == 8 && topk_group == 4 && experts == 256) ||
                     (num_expert_group == 1 && topk_group == 1 && (experts == 160 || experts == 320 || experts == 384 || experts == 448));
  TORCH_CHECK(known, "Invalid arguments with TOPK = ", topk, ", NUM_EXPERT_GROUP = ", num_expert_group, ", TOPK_GROUP = ", topk_group,
              ", NUM_EXPERTS = ", experts);
  TORCH_CHECK(correction_bias.numel() == experts);
  TORCH_CHECK(out_routing_weights.numel() == tokens * topk && out_selected_experts.numel() == tokens * topk);
  const c10::cuda::OptionalCUDAGuard guard(device_of(gating_outputs));
  check_rc(mcop_moe_gate_grouped_sigmoid_shared(gating_outputs.data_ptr(), correction_bias.data_ptr(), out_routing_weights.data_ptr<float>(),
                                                out_selected_experts.data_ptr<int32_t>(), tokens, (int)experts, (int)num_expert_group,
                                                (int)topk_group, (int)topk, renormalize ? 1 : 0, (int)num_shared,
                                                routed_scaling_factor.value_or(1.0), dtype_code(gating_outputs, "gating_outputs"),
                                                cur_stream()));
  return 0;
}

// mcoplib.op.moe_scatter_dynamic_quant (op/moe_scatter_dynamic_quant.cu:312-341)
void moe_scatter_dynamic_quant(Tensor hidden_status, Tensor selected_experts, Tensor moe_weights, Tensor smooth_scale, Tensor scatter_tokens,
                               Tensor scatter_per_token_scale, Tensor scatter_tokens_offset, Tensor experts_token_count,
                               Tensor experts_token_start, int experts_per_rank, int shared_experts_per_rank, int shared_tokens_per_sp,
                               std::optional<Tensor> tok2row) {
  MCOP_DEBUG_CALL("moe_scatter_dynamic_quant", hidden_status, selected_experts, moe_weights, smooth_scale, scatter_tokens, scatter_per_token_scale, scatter_tokens_offset, experts_token_count, experts_token_start, experts_per_rank, shared_experts_per_rank, shared_tokens_per_sp, tok2row);
  check_cuda(hidden_status, "hidden_status"); check_cuda(selected_experts, "selected_experts"); check_cuda(smooth_scale, "smooth_scale");
  TORCH_CHECK(hidden_status.is_contiguous() && selected_experts.is_contiguous() && smooth_scale.is_contiguous());
  TORCH_CHECK(hidden_status.scalar_type() == at::kBFloat16, "Only float16, bfloat16 are supported");
  TORCH_CHECK(shared_experts_per_rank == 0 && shared_tokens_per_sp == 0, "shared experts are not built");
  TORCH_CHECK(experts_per_rank <= 256, "Unsupported, num_experts_per_rank should less than or equal to 256");
  TORCH_CHECK(selected_experts.scalar_type() == at::kInt && moe_weights.scalar_type() == at::kFloat && smooth_scale.scalar_type() == at::kFloat);
  TORCH_CHECK(scatter_tokens.scalar_type() == at::kChar && scatter_per_token_scale.scalar_type() == at::kFloat &&
              scatter_tokens_offset.scalar_type() == at::kInt && experts_token_count.scalar_type() == at::kInt &&
              experts_token_start.scalar_type() == at::kInt);
  TORCH_CHECK(moe_weights.is_contiguous() && scatter_tokens.is_contiguous() && scatter_per_token_scale.is_contiguous() &&
              scatter_tokens_offset.is_contiguous() && experts_token_count.is_contiguous() && experts_token_start.is_contiguous());
  const int64_t hidden = hidden_status.size(-1);
  const int64_t tokens = hidden ? hidden_status.numel() / hidden : 0;
  const int topk = (int)selected_experts.size(-1);
  TORCH_CHECK(selected_experts.numel() == tokens * topk && moe_weights.numel() == tokens * topk);
  TORCH_CHECK(smooth_scale.numel() >= (int64_t)experts_per_rank * hidden);
  TORCH_CHECK(scatter_tokens.numel() >= tokens * topk * hidden && scatter_per_token_scale.numel() >= tokens * topk &&
              scatter_tokens_offset.numel() >= tokens * topk);
  TORCH_CHECK(experts_token_count.numel() >= experts_per_rank && experts_token_start.numel() >= experts_per_rank);
  int32_t* t2r = nullptr;
  if (tok2row.has_value()) {
    TORCH_CHECK(tok2row->scalar_type() == at::kInt && tok2row->is_contiguous() && tok2row->numel() == tokens * topk);
    t2r = tok2row->data_ptr<int32_t>();
  }
  const c10::cuda::OptionalCUDAGuard guard(device_of(hidden_status));
  const size_t ws_bytes = mcop_moe_scatter_workspace_bytes(tokens, topk, experts_per_rank);
  Tensor ws = scratch_bytes(ws_bytes, hidden_status);
  check_rc(mcop_moe_scatter_quant_i8(hidden_status.data_ptr(), selected_experts.data_ptr<int32_t>(), moe_weights.data_ptr<float>(),
                                     smooth_scale.data_ptr<float>(), scatter_tokens.data_ptr<int8_t>(), scatter_per_token_scale.data_ptr<float>(),
                                     scatter_tokens_offset.data_ptr<int32_t>(), experts_token_count.data_ptr<int32_t>(),
                                     experts_token_start.data_ptr<int32_t>(), t2r, tokens, hidden, topk, experts_per_rank, ws.data_ptr(),
                                     (size_t)ws.numel(), cur_stream()));
}

// mcoplib.op.moe_gather (op/moe_gather.cu:137-150)
void moe_gather(Tensor scatter_tokens, Tensor scatter_tokens_offset, Tensor convergent_tokens, std::optional<Tensor> tok2row) {
  MCOP_DEBUG_CALL("moe_gather", scatter_tokens, scatter_tokens_offset, convergent_tokens, tok2row);
  check_cuda(scatter_tokens, "scatter_tokens");
  TORCH_CHECK(scatter_tokens.scalar_type() == at::kBFloat16 && convergent_tokens.scalar_type() == at::kBFloat16,
              "Only float16, bfloat16 are supported");
  TORCH_CHECK(scatter_tokens.is_contiguous() && scatter_tokens_offset.is_contiguous() && convergent_tokens.is_contiguous());
  TORCH_CHECK(scatter_tokens_offset.scalar_type() == at::kInt);
  const int64_t hidden = scatter_tokens.size(-1);
  const int64_t rows = hidden ? scatter_tokens.numel() / hidden : 0;
  TORCH_CHECK(convergent_tokens.size(-1) == hidden);
  const int64_t tokens = hidden ? convergent_tokens.numel() / hidden : 0;
  TORCH_CHECK(scatter_tokens_offset.numel() >= rows);
  const c10::cuda::OptionalCUDAGuard guard(device_of(scatter_tokens));
  const int32_t* t2r = nullptr;
  int topk = 0;
  Tensor ws;
  void* wsp = nullptr;
  size_t ws_bytes = 0;
  if (tok2row.has_value()) {
    TORCH_CHECK(tok2row->scalar_type() == at::kInt && tok2row->is_contiguous() && tok2row->dim() == 2 && tok2row->size(0) == tokens);
    t2r = tok2row->data_ptr<int32_t>();
    topk = (int)tok2row->size(1);
  } else {
    ws_bytes = mcop_moe_gather_workspace_bytes(tokens, rows);
    ws = scratch_bytes(ws_bytes, scatter_tokens);
    wsp = ws.data_ptr();
    ws_bytes = (size_t)ws.numel();
  }
  check_rc(mcop_moe_gather(scatter_tokens.data_ptr(), scatter_tokens_offset.data_ptr<int32_t>(), convergent_tokens.data_ptr(), t2r, topk,
                           tokens, rows, hidden, wsp, ws_bytes, cur_stream()));
}

// mcoplib.op.moe_swiglu_dynamic_quantize (op/moe_swiglu_dq.cu, include/moe_swiglu_dq.h)
void moe_swiglu_dynamic_quantize(Tensor scatter_tokens, Tensor smooth_scale, Tensor experts_tokens_start, Tensor experts_tokens_count,
                                 Tensor& y, Tensor& per_tokens_scale, int total_experts_num) {
  MCOP_DEBUG_CALL("moe_swiglu_dynamic_quantize", scatter_tokens, smooth_scale, experts_tokens_start, experts_tokens_count, y, per_tokens_scale, total_experts_num);
  check_cuda(scatter_tokens, "scatter_tokens");
  TORCH_CHECK(scatter_tokens.scalar_type() == at::kBFloat16, "Only bfloat16 is supported");
  TORCH_CHECK(scatter_tokens.is_contiguous() && smooth_scale.is_contiguous() && y.is_contiguous() && per_tokens_scale.is_contiguous());
  TORCH_CHECK(experts_tokens_start.is_contiguous() && experts_tokens_count.is_contiguous());
  TORCH_CHECK(smooth_scale.scalar_type() == at::kFloat && y.scalar_type() == at::kChar && per_tokens_scale.scalar_type() == at::kFloat);
  TORCH_CHECK(experts_tokens_start.scalar_type() == at::kInt && experts_tokens_count.scalar_type() == at::kInt);
  const int64_t hidden2 = scatter_tokens.size(-1);
  TORCH_CHECK(hidden2 % 2 == 0, "the last dimension holds gate || up");
  const int64_t hidden = hidden2 / 2;
  const int64_t rows = hidden2 ? scatter_tokens.numel() / hidden2 : 0;
  TORCH_CHECK(y.numel() == rows * hidden && per_tokens_scale.numel() >= rows);
  TORCH_CHECK(total_experts_num >= 1 && experts_tokens_start.numel() >= total_experts_num && experts_tokens_count.numel() >= total_experts_num);
  TORCH_CHECK(smooth_scale.numel() >= (int64_t)total_experts_num * hidden);
  const c10::cuda::OptionalCUDAGuard guard(device_of(scatter_tokens));
  check_rc(mcop_moe_swiglu_quant_i8(scatter_tokens.data_ptr(), smooth_scale.data_ptr<float>(), experts_tokens_start.data_ptr<int32_t>(),
                                    experts_tokens_count.data_ptr<int32_t>(), y.data_ptr<int8_t>(), per_tokens_scale.data_ptr<float>(), rows,
                                    hidden, total_experts_num, cur_stream()));
}

// mcoplib.op.fused_add_rms_norm_dynamic_per_token_quant_padding_output
// (op/fused_add_layernorm_per_token_quant_padding_output.cu:397-416): `output` is the int8 view of a
// [tokens, pad_size] 16-bit tensor, i.e. int8 [tokens, 2 * pad_size]
void fused_add_rms_norm_dynamic_per_token_quant_padding_output(Tensor& output, Tensor& output_rms, Tensor& output_quant_int8,
                                                               Tensor& out_scales, const Tensor& input, Tensor& residual,
                                                               const Tensor& weight, int64_t pad_size, double epsilon) {
  MCOP_DEBUG_CALL("add_rms_norm_dynamic_per_token_quant_padding_output", output, output_rms, output_quant_int8, out_scales, input, residual, weight, pad_size, epsilon);
  check_cuda(input, "input");
  TORCH_CHECK(output.dtype() == torch::kInt8);
  TORCH_CHECK(input.dtype() == at::ScalarType::BFloat16);
  TORCH_CHECK(output.is_contiguous() && input.is_contiguous());
  TORCH_CHECK(residual.is_contiguous() && weight.is_contiguous() && output_rms.is_contiguous() && output_quant_int8.is_contiguous() &&
              out_scales.is_contiguous());
  TORCH_CHECK(residual.scalar_type() == input.scalar_type() && weight.scalar_type() == input.scalar_type() &&
              output_rms.scalar_type() == input.scalar_type());
  TORCH_CHECK(output_quant_int8.scalar_type() == at::kChar && out_scales.scalar_type() == at::kFloat);
  const int64_t hidden = input.size(-1);
  TORCH_CHECK(hidden > 0 && hidden % 4 == 0, "hidden size must be a multiple of 4");
  const int64_t tokens = input.numel() / hidden;
  TORCH_CHECK(residual.numel() == input.numel() && weight.numel() == hidden && output_rms.numel() == input.numel() &&
              output_quant_int8.numel() == input.numel() && out_scales.numel() >= tokens);
  TORCH_CHECK(pad_size * 2 >= hidden + 4 && output.numel() == tokens * pad_size * 2,
              "output must be the int8 view of [tokens, pad_size] 16-bit elements and hold the codes and the scale");
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_add_rmsnorm_quant_i8_padded(input.data_ptr(), residual.data_ptr(), weight.data_ptr(), output.data_ptr(),
                                            output_rms.data_ptr(), output_quant_int8.data_ptr<int8_t>(), out_scales.data_ptr<float>(),
                                            tokens, hidden, pad_size, (float)epsilon, 0,
                                            dtype_code(input, "fused_add_rms_norm_dynamic_per_token_quant_padding_output"), cur_stream()));
}

// mcoplib.op.fused_silu_mul_dq_reorder_quant (op/int8_quant_kernels.cu:1893-1940, include/int8_quant_kernel.h:7-14).
// w2_scale is accepted and, as in the reference (HAS_SCALE = false in every instantiation), not applied.
void fused_silu_mul_dq_reorder_quant(Tensor& out, Tensor& scale, const Tensor& input, const Tensor& reorder_topk_ids,
                                     const Tensor& w2_scale, int64_t start_expert_id, int64_t end_expert_id) {
  MCOP_DEBUG_CALL("fused_silu_mul_dq_quant_reordered_topk_interface", out, scale, input, reorder_topk_ids, w2_scale, start_expert_id, end_expert_id);
  check_cuda(input, "input");
  TORCH_CHECK(input.is_contiguous());
  TORCH_CHECK(scale.is_contiguous());
  TORCH_CHECK(out.is_contiguous());
  TORCH_CHECK(reorder_topk_ids.is_contiguous());
  TORCH_CHECK(out.scalar_type() == at::kChar && scale.scalar_type() == at::kFloat);
  TORCH_CHECK(reorder_topk_ids.scalar_type() == at::kInt || reorder_topk_ids.scalar_type() == at::kLong,
              "reorder_topk_ids must be int32 or int64");
  (void)w2_scale;
  const int64_t hidden2 = input.size(-1);
  TORCH_CHECK(hidden2 > 0 && hidden2 % 2 == 0, "the last dimension holds gate || up");
  const int64_t rows = input.numel() / hidden2;
  TORCH_CHECK(out.numel() == rows * (hidden2 / 2) && scale.numel() >= rows && reorder_topk_ids.numel() >= rows);
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_silu_mul_quant_i8(input.data_ptr(), dtype_code(input, "fused_silu_mul_dq_reorder_quant"), reorder_topk_ids.data_ptr(),
                                  reorder_topk_ids.scalar_type() == at::kLong ? 1 : 0, start_expert_id, end_expert_id,
                                  out.data_ptr<int8_t>(), scale.data_ptr<float>(), rows, hidden2 / 2, cur_stream()));
}

// sglang's fused_silu_mul_dq_quant_interface (op/int8_quant_kernels.cu:1877-1891): every row is processed
void fused_silu_mul_dq_quant(Tensor& out, Tensor& scale, const Tensor& input) {
  MCOP_DEBUG_CALL("fused_silu_mul_dq_quant_interface", out, scale, input);
  check_cuda(input, "input");
  TORCH_CHECK(input.is_contiguous());
  TORCH_CHECK(scale.is_contiguous());
  TORCH_CHECK(out.is_contiguous());
  TORCH_CHECK(out.scalar_type() == at::kChar && scale.scalar_type() == at::kFloat);
  const int64_t hidden2 = input.size(-1);
  TORCH_CHECK(hidden2 > 0 && hidden2 % 2 == 0, "the last dimension holds gate || up");
  const int64_t rows = input.numel() / hidden2;
  TORCH_CHECK(out.numel() == rows * (hidden2 / 2) && scale.numel() >= rows);
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_silu_mul_quant_i8(input.data_ptr(), dtype_code(input, "fused_silu_mul_dq_quant"), nullptr, 0, 0, 0, out.data_ptr<int8_t>(),
                                  scale.data_ptr<float>(), rows, hidden2 / 2, cur_stream()));
}

// mcoplib.op.fused_silu_mul_dq_mask_quant (op/int8_quant_kernels.cu:1844-1875, include/int8_quant_kernel.h:2-5)
void fused_silu_mul_dq_mask_quant(Tensor& out, const Tensor& input, const Tensor& mask) {
  MCOP_DEBUG_CALL("fused_silu_mul_dq_mask_quant_pack", out, input, mask);
  check_cuda(input, "input");
  TORCH_CHECK(input.is_contiguous());
  TORCH_CHECK(out.is_contiguous());
  TORCH_CHECK(mask.is_contiguous());
  TORCH_CHECK(out.scalar_type() == input.scalar_type(), "out is a byte record per row, declared in the activation dtype");
  TORCH_CHECK(mask.scalar_type() == at::kInt || mask.scalar_type() == at::kLong, "mask must be int32 or int64");
  const int64_t hidden2 = input.size(-1);
  TORCH_CHECK(hidden2 > 0 && hidden2 % 2 == 0, "the last dimension holds gate || up");
  const int64_t rows = input.numel() / hidden2;
  const int64_t groups = mask.numel();
  TORCH_CHECK(groups >= 1 && groups <= 1024 && rows % groups == 0);
  const int64_t out_stride = ((hidden2 / 4 + 2) + 255) / 256 * 256;
  TORCH_CHECK(out.numel() >= rows * out_stride && out.size(-1) == out_stride, "out must be [groups, rows, ", out_stride, "]");
  const c10::cuda::OptionalCUDAGuard guard(device_of(input));
  check_rc(mcop_silu_mul_quant_i8_masked_pack(input.data_ptr(), dtype_code(input, "fused_silu_mul_dq_mask_quant"), mask.data_ptr(),
                                              mask.scalar_type() == at::kLong ? 1 : 0, out.data_ptr(), groups, rows / groups, hidden2 / 2,
                                              out_stride, cur_stream()));
}

// Weighted combine (addition of this build)
void moe_gather_weighted(Tensor y, Tensor row2tok, Tensor topk_ids, Tensor topk_weights, Tensor experts_token_start, Tensor out,
                         bool accumulate, std::optional<Tensor> tok2row) {
  MCOP_DEBUG_CALL("moe_gather_weighted", y, row2tok, topk_ids, topk_weights, experts_token_start, out, accumulate, tok2row);
  check_cuda(y, "y");
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "Only bfloat16 is supported");
  TORCH_CHECK(y.is_contiguous() && row2tok.is_contiguous() && topk_ids.is_contiguous() && topk_weights.is_contiguous() &&
              experts_token_start.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(row2tok.scalar_type() == at::kInt && topk_ids.scalar_type() == at::kInt && topk_weights.scalar_type() == at::kFloat &&
              experts_token_start.scalar_type() == at::kInt);
  const int64_t hidden = y.size(-1);
  const int64_t rows = hidden ? y.numel() / hidden : 0;
  const int64_t tokens = hidden ? out.numel() / hidden : 0;
  const int topk = (int)topk_ids.size(-1);
  TORCH_CHECK(out.size(-1) == hidden && topk_ids.numel() == tokens * topk && topk_weights.numel() == tokens * topk && row2tok.numel() >= rows);
  const c10::cuda::OptionalCUDAGuard guard(device_of(y));
  const int32_t* t2r = nullptr;
  Tensor ws;
  void* wsp = nullptr;
  size_t ws_bytes = 0;
  if (tok2row.has_value()) {
    TORCH_CHECK(tok2row->scalar_type() == at::kInt && tok2row->is_contiguous() && tok2row->numel() == tokens * topk);
    t2r = tok2row->data_ptr<int32_t>();
  } else {
    ws_bytes = mcop_moe_gather_workspace_bytes(tokens, rows);
    ws = scratch_bytes(ws_bytes, y);
    wsp = ws.data_ptr();
    ws_bytes = (size_t)ws.numel();
  }
  check_rc(mcop_moe_gather_weighted(y.data_ptr(), row2tok.data_ptr<int32_t>(), topk_ids.data_ptr<int32_t>(), topk_weights.data_ptr<float>(),
                                    experts_token_start.data_ptr<int32_t>(), out.data_ptr(), t2r, accumulate ? 1 : 0, tokens, rows, hidden,
                                    topk, (int)experts_token_start.numel(), wsp, ws_bytes, cur_stream()));
}

}  // namespace

// ---------------------------------------------------------------- registration

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.doc() = "mcoplib.op operator surface of the per-token inference hot path, B200 (sm_100a) kernels";
  m.def("rms_norm_dynamic_per_token_quant", &rms_norm_dynamic_per_token_quant_9);
  m.def("rms_norm_dynamic_per_token_quant_custom", &rms_norm_dynamic_per_token_quant_vllm);
  m.def("sgl_rms_norm_dynamic_per_token_quant_custom", &rms_norm_dynamic_per_token_quant_sgl);
  m.def("rms_norm", &rms_norm);
  m.def("head_rms_norm", &head_rms_norm);
  m.def("scale_dynamic_quant", &scale_dynamic_quant, py::arg("hidden_states"), py::arg("smooth_scales"),
        py::arg("dst_torch_dtype") = at::ScalarType::Char);
  m.def("rotary_embedding", &rotary_embedding_packed, py::arg("packed_qkv"), py::arg("q_len"), py::arg("accum_q_lens"),
        py::arg("cache_lens"), py::arg("cos"), py::arg("sin"), py::arg("output"), py::arg("q_head_num"), py::arg("kv_head_num"),
        py::arg("rope_offset") = 0);
  m.def("fused_rope_fwd", &fused_rope_fwd, py::arg("qkv"), py::arg("cos"), py::arg("sin"), py::arg("indexes"),
        py::arg("force_bf16_attn") = false);
  m.def("fused_rope_bwd", &fused_rope_bwd, py::arg("qkv"), py::arg("cos"), py::arg("sin"), py::arg("indexes"),
        py::arg("force_bf16_attn") = false);
  m.def("store_kv_cache_cuda_interface", &store_kv_cache_cuda_interface);
  m.def("moe_sum", &moe_sum, py::arg("input"), py::arg("output"));
  m.def("moe_sum_reduce", &moe_sum_reduce, py::arg("input"), py::arg("output"), py::arg("routed_scaling_factor"));
  m.def("moe_align_block_size", &moe_align_block_size, py::arg("topk_ids"), py::arg("num_experts"), py::arg("block_size"),
        py::arg("sorted_token_ids"), py::arg("experts_ids"), py::arg("num_tokens_post_pad"), py::arg("maybe_expert_map") = py::none());
  m.def("moe_softmax_topk", &moe_softmax_topk);
  m.def("fused_moe_gate_deepseek", &fused_moe_gate_deepseek, py::arg("gating_outputs"), py::arg("correction_bias"),
        py::arg("out_routing_weights"), py::arg("out_selected_experts"), py::arg("topk"), py::arg("renormalize"),
        py::arg("num_expert_group"), py::arg("topk_group"), py::arg("num_fused_shared_experts") = py::none(),
        py::arg("routed_scaling_factor") = py::none(), py::arg("moegate_type") = py::none(), py::arg("debug_group_mask") = py::none());
  m.def("fused_moe_gate_opt", &fused_moe_gate_opt, py::arg("gating_outputs"), py::arg("correction_bias"), py::arg("out_routing_weights"),
        py::arg("out_selected_experts"), py::arg("topk"), py::arg("renormalize"), py::arg("num_expert_group"), py::arg("topk_group"),
        py::arg("num_fused_shared_experts") = py::none(), py::arg("routed_scaling_factor") = py::none());
  m.def("moe_scatter_dynamic_quant", &moe_scatter_dynamic_quant, py::arg("hidden_status"), py::arg("selected_experts"),
        py::arg("moe_weights"), py::arg("smooth_scale"), py::arg("scatter_tokens"), py::arg("scatter_per_token_scale"),
        py::arg("scatter_tokens_offset"), py::arg("experts_token_count"), py::arg("experts_token_start"), py::arg("experts_per_rank"),
        py::arg("shared_experts_per_rank"), py::arg("shared_tokens_per_sp"), py::arg("tok2row") = py::none());
  m.def("moe_gather", &moe_gather, py::arg("scatter_tokens"), py::arg("scatter_tokens_offset"), py::arg("convergent_tokens"),
        py::arg("tok2row") = py::none());
  m.def("moe_swiglu_dynamic_quantize", &moe_swiglu_dynamic_quantize);
  m.def("fused_add_rms_norm_dynamic_per_token_quant_padding_output", &fused_add_rms_norm_dynamic_per_token_quant_padding_output);
  m.def("fused_silu_mul_dq_mask_quant", &fused_silu_mul_dq_mask_quant);
  m.def("fused_silu_mul_dq_reorder_quant", &fused_silu_mul_dq_reorder_quant);
  m.def("fused_silu_mul_dq_quant", &fused_silu_mul_dq_quant);
  // additions of this build (no reference counterpart)
  m.def("rope_kv_store_int8", &rope_kv_store_int8);
  m.def("moe_gather_weighted", &moe_gather_weighted, py::arg("y"), py::arg("row2tok"), py::arg("topk_ids"), py::arg("topk_weights"),
        py::arg("experts_token_start"), py::arg("out"), py::arg("accumulate"), py::arg("tok2row") = py::none());
  // torch-library functions also reachable directly (same objects the dispatcher calls)
  m.def("fused_add_rms_norm", &fused_add_rms_norm);
  m.def("vllm_rotary_embedding", &rotary_embedding_vllm);
  m.def("reshape_and_cache_flash", &reshape_and_cache_flash);
  m.def("reshape_and_cache", &reshape_and_cache);
  m.def("store_kv_cache", &store_kv_cache);
  m.def("apply_rope_pos_ids_cos_sin_cache", &apply_rope_pos_ids_cos_sin_cache, py::arg("q"), py::arg("k"), py::arg("q_rope"),
        py::arg("k_rope"), py::arg("cos_sin_cache"), py::arg("pos_ids"), py::arg("interleave"), py::arg("enable_pdl") = false,
        py::arg("v") = py::none(), py::arg("k_buffer") = py::none(), py::arg("v_buffer") = py::none(), py::arg("kv_cache_loc") = py::none());
  m.def("topk_softmax", &topk_softmax);
  m.def("grouped_topk", &grouped_topk, py::arg("scores"), py::arg("n_group"), py::arg("topk_group"), py::arg("topk"),
        py::arg("renormalize"), py::arg("routed_scaling_factor"), py::arg("bias"), py::arg("scoring_func") = 0);
  m.def("dynamic_scaled_int8_quant", &dynamic_scaled_int8_quant);
#define MCOP_STR_(x) #x
#define MCOP_STR(x) MCOP_STR_(x)
  m.attr("torch_namespace") = MCOP_STR(MCOP_TORCH_NS);
  m.attr("torch_moe_namespace") = MCOP_STR(MCOP_TORCH_NS_MOE);
}

TORCH_LIBRARY(MCOP_TORCH_NS, ops) {
  ops.def("fused_add_rms_norm(Tensor! input, Tensor! residual, Tensor weight, float epsilon) -> ()");
  ops.impl("fused_add_rms_norm", torch::kCUDA, &fused_add_rms_norm);
  ops.def(
      "rms_norm_dynamic_per_token_quant(Tensor! result, Tensor input, Tensor weight, Tensor! scale, float epsilon, "
      "Tensor? scale_ub, Tensor!? residual) -> ()");
  ops.impl("rms_norm_dynamic_per_token_quant", torch::kCUDA, &rms_norm_dynamic_per_token_quant_C);
  ops.def("dynamic_scaled_int8_quant(Tensor! result, Tensor input, Tensor! scale, Tensor!? azp) -> ()");
  ops.impl("dynamic_scaled_int8_quant", torch::kCUDA, &dynamic_scaled_int8_quant);
  ops.def(
      "rotary_embedding(Tensor positions, Tensor! query, Tensor!? key, int head_size, Tensor cos_sin_cache, bool is_neox) -> ()");
  ops.impl("rotary_embedding", torch::kCUDA, &rotary_embedding_vllm);
  ops.def(
      "rope_kv_store_int8(Tensor positions, Tensor! query, Tensor! key, Tensor value, int head_size, Tensor cos_sin_cache, "
      "bool is_neox, Tensor! key_cache, Tensor! value_cache, Tensor slot_mapping, Tensor k_scale, Tensor v_scale) -> ()");
  ops.impl("rope_kv_store_int8", torch::kCUDA, &rope_kv_store_int8);
}

TORCH_LIBRARY(MCOP_TORCH_NS_MOE, moe_ops) {
  moe_ops.def(
      "topk_softmax(Tensor! topk_weights, Tensor! topk_indices, Tensor! token_expert_indices, Tensor gating_output, "
      "bool renormalize) -> ()");
  moe_ops.impl("topk_softmax", torch::kCUDA, &topk_softmax);
  moe_ops.def(
      "grouped_topk(Tensor scores, int n_group, int topk_group, int topk, bool renormalize, float routed_scaling_factor, "
      "Tensor bias, int scoring_func) -> (Tensor, Tensor)");
  moe_ops.impl("grouped_topk", torch::kCUDA, &grouped_topk);
  moe_ops.def("moe_sum(Tensor input, Tensor! output) -> ()");
  moe_ops.impl("moe_sum", torch::kCUDA, &moe_sum);
  moe_ops.def(
      "moe_align_block_size(Tensor topk_ids, int num_experts, int block_size, Tensor! sorted_token_ids, Tensor! experts_ids, "
      "Tensor! num_tokens_post_pad, Tensor? maybe_expert_map) -> ()");
  moe_ops.impl("moe_align_block_size", torch::kCUDA, &moe_align_block_size);
}

TORCH_LIBRARY(MCOP_TORCH_NS_CACHE, cache_ops) {
  cache_ops.def(
      "reshape_and_cache(Tensor key, Tensor value, Tensor! key_cache, Tensor! value_cache, Tensor slot_mapping, "
      "str kv_cache_dtype, Tensor k_scale, Tensor v_scale) -> ()");
  cache_ops.impl("reshape_and_cache", torch::kCUDA, &reshape_and_cache);
  cache_ops.def(
      "reshape_and_cache_flash(Tensor key, Tensor value, Tensor! key_cache, Tensor! value_cache, Tensor slot_mapping, "
      "str kv_cache_dtype, Tensor k_scale, Tensor v_scale) -> ()");
  cache_ops.impl("reshape_and_cache_flash", torch::kCUDA, &reshape_and_cache_flash);
}
