/*
 * mcop_b200 - C ABI of the B200 (sm_100a) implementation of mcoplib's per-token inference hot path.
 *
 * Every entry point takes raw DEVICE pointers, 64-bit sizes/strides and a CUDA stream, enqueues its
 * kernels on that stream and returns at once:
 *     0  (MCOP_OK)          launched
 *    <0                     rejected before any launch (see the enum); mcop_last_error() has the text.
 * No entry point allocates, frees or synchronises unless its comment says so.  Buffers are owned by the
 * caller.  Entry points are safe to call from several host threads; the error text is per thread.
 *
 * Each declaration cites the operator of MetaX-MACA/mcoplib it replaces (path:line inside that project).
 * Element type codes: MCOP_F32 / MCOP_BF16 / MCOP_F16.
 */
#ifndef MCOP_B200_H_
#define MCOP_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* mcop_stream_t; /* == cudaStream_t */

enum { MCOP_F32 = 0, MCOP_BF16 = 1, MCOP_F16 = 2 };

enum {
  MCOP_OK = 0,
  MCOP_ERR_ARGUMENT = -1,    /* null pointer, negative size, bad stride or misaligned buffer */
  MCOP_ERR_UNSUPPORTED = -2, /* a shape / dtype combination this build has no kernel for */
  MCOP_ERR_WORKSPACE = -3,   /* workspace missing or too small */
  MCOP_ERR_CUDA = -4         /* the launch itself was refused by the CUDA runtime */
};

/* Library version (major*10000 + minor*100 + patch). */
int mcop_version(void);
/* Text of the last error on the calling thread ("" if none). */
const char* mcop_last_error(void);
/* Device-side status of the current device: one word per device that kernels set and the host reads.
 *   - the row-pipeline kernels bound every wait on an asynchronous copy; a kernel whose wait runs out records
 *     MCOP_DEVERR_WAIT_FIRST .. MCOP_DEVERR_WAIT_LAST (which wait it was: 1 / 2 norm + quant row wait / drain, 3 / 4 gather,
 *     5 / 6 scatter, 7 RoPE, 11 / 12 scale_dynamic_quant, 13 / 14 head_rms_norm), stops issuing copies, drains those in
 *     flight and returns instead of hanging;
 *   - a value read from a caller's tensor is never turned into an address unchecked: a position outside the
 *     cos / sin table, a cache slot or cache position outside the cache make the kernel SKIP that token (nothing of
 *     it is read through the bad index, nothing is written for it) and record MCOP_DEVERR_POSITION / _SLOT / _KV_INDEX.
 * The first code recorded wins.  Entry points return MCOP_OK when they have launched, so a caller that wants to know
 * calls this after synchronising: it returns the code (0 = none) and clears it, or a negative MCOP_ERR_*.
 * SYNCHRONISES with the device.  No counterpart in the reference (its kernels neither wait nor check). */
int mcop_device_error(void);
enum {
  MCOP_DEVERR_WAIT_FIRST = 1,
  MCOP_DEVERR_WAIT_LAST = 15,
  MCOP_DEVERR_POSITION = 16, /* RoPE position outside [0, max_position) */
  MCOP_DEVERR_SLOT = 17,     /* paged-cache slot >= num_blocks * block_size */
  MCOP_DEVERR_KV_INDEX = 18, /* store_kv: slot id outside [0, num_slots) or cache position outside [0, max_len) */
  MCOP_DEVERR_SELFTEST = 99  /* recorded by mcop_selftest_wait_timeout */
};

/* Self-test of the bounded-wait path; no counterpart in the reference.  Launches ONE small CTA that arms a ring stage
 * for `bytes` bytes WITHOUT issuing any copy for it (nothing is in flight, nothing can land late), waits for it with a
 * limit of `spin_limit` tries (1 .. 1 << 20), records MCOP_DEVERR_SELFTEST in the error word when the wait runs out -
 * which it must - runs the same drain the pipeline kernels run, and returns.  The kernel neither faults nor hangs and
 * the context stays usable; mcop_device_error() then yields MCOP_DEVERR_SELFTEST once and 0 afterwards. */
int mcop_selftest_wait_timeout(int spin_limit, mcop_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Part 1 - residual add + RMSNorm (+ per-token int8 quantisation)
 * ---------------------------------------------------------------------------------------------- */

/* torch.ops._C.fused_add_rms_norm, op/vllm/layernorm_kernels.cu:243-292 (schema op/vllm/torch_bindings.cpp:161-164).
 * In place: r = T(x + res); res := r; x := T(T(r * rsqrt(mean(r^2)+eps)) * w).
 * x [tokens, hidden] with row stride x_row_stride (elements); residual, weight contiguous. */
int mcop_fused_add_rmsnorm(void* x, int64_t x_row_stride, void* residual, const void* weight,
                           int64_t tokens, int64_t hidden, float eps, int dtype, mcop_stream_t stream);

/* torch.ops._C.rms_norm_dynamic_per_token_quant,
 * op/vllm/quantization/fused_kernels/fused_layernorm_dynamic_per_token_quant.cu:163-192 (schema torch_bindings.cpp:216-221),
 * and mcoplib.op.rms_norm_dynamic_per_token_quant_custom, op/rms_norm_dynamic_per_token_quant.cu:266-285.
 * s = x (+ res); res := T(s) (if residual != NULL); n = T(T(s * rsqrt(mean(s^2)+eps)) * w);
 * scale = max(min(max|n|, *scale_ub) / 127, FLT_EPSILON); out = int8(rne(n * (1/scale))).
 * out [tokens, hidden] int8, scales [tokens] fp32, scale_ub NULL or one fp32 on the device. */
int mcop_add_rmsnorm_quant_i8(int8_t* out, float* scales, const void* x, int64_t x_row_stride,
                              const void* weight, void* residual, const float* scale_ub,
                              int64_t tokens, int64_t hidden, float eps, int dtype, mcop_stream_t stream);

/* mcoplib.op.rms_norm_dynamic_per_token_quant (9 arguments), op/fused_rms_norm_dq.cu:646-667
 * (include/fused_rms_norm_dq.h:3-12).  Keeps the reference's convention of DIVIDING by rsqrt(mean+eps):
 * after_res = T(x + res); after_norm = T(after_res / r * w); y = after_res / r * w * smooth;
 * scales = max|y| / 127; out = int8(rne(y / scale)) clamped to +-127.  weight and smooth share wdtype
 * (MCOP_BF16 or MCOP_F32).  residual may be NULL; after_res and after_norm are always written. */
int mcop_rmsnorm_smooth_quant_i8(int8_t* out, float* scales, void* after_res, void* after_norm,
                                 const void* x, const void* weight, const void* smooth, const void* residual,
                                 int64_t tokens, int64_t hidden, float eps, int dtype, int wdtype,
                                 mcop_stream_t stream);

/* mcoplib.op.rms_norm, op/fused_rms_norm_dq.cu:980-999 (include/fused_rms_norm_dq.h:16-24).
 * out = T((x [+ res]) * d * w), d = rsqrt(mean+eps) or, with rms_div != 0, 1/rsqrt(mean+eps).
 * residual and after_res are both NULL or both set (after_res = T(x + res)). */
int mcop_rmsnorm(void* out, const void* x, const void* weight, void* after_res, const void* residual,
                 int64_t tokens, int64_t hidden, float eps, int rms_div, int dtype, int wdtype,
                 mcop_stream_t stream);

/* mcoplib.op.head_rms_norm, op/fused_rms_norm_dq.cu:804-812: per-head RMSNorm (divide-by-rsqrt form) of
 * heads [head_offset, head_offset + head_norm) of x [tokens, heads, head_dim] into out (same layout; other
 * heads of out are not touched); weight [heads, head_dim] in wdtype. */
int mcop_head_rmsnorm(void* out, const void* x, const void* weight, int64_t tokens, int64_t heads,
                      int64_t head_dim, float eps, int head_offset, int head_norm, int dtype, int wdtype,
                      mcop_stream_t stream);

/* mcoplib.op.scale_dynamic_quant, op/scale_dynamic_quant.cu:127-153: y = x * smooth (fp32 smooth [hidden]);
 * scales = max|y| / 127; out = int8(rne(y / scale)).  The caller allocates out and scales. */
int mcop_scale_dynamic_quant_i8(int8_t* out, float* scales, const void* x, const float* smooth,
                                int64_t tokens, int64_t hidden, int dtype, mcop_stream_t stream);

/* torch.ops._C.dynamic_scaled_int8_quant (symmetric form, azp = None),
 * op/vllm/quantization/compressed_tensors/int8_quant_kernels.cu:95-132 (schema op/vllm/torch_bindings.cpp:375-379):
 * scales = max|x| / 127; out = int8(rne(x * (127 / max|x|))), all-zero rows give codes 0. */
int mcop_dynamic_scaled_int8_quant(int8_t* out, float* scales, const void* x, int64_t tokens, int64_t hidden,
                                   int dtype, mcop_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Part 2 - rotary embedding and the int8 KV-cache store
 * ---------------------------------------------------------------------------------------------- */

/* torch.ops._C.rotary_embedding, op/vllm/pos_encoding_kernels.cu:135-217 (schema torch_bindings.cpp:233-237).
 * In-place RoPE of query (and key unless NULL).  cos_sin_cache [max_position, rot_dim] = cos || sin, in the
 * activation dtype (arithmetic in T, rounded after every operation) or in fp32 (fp32 arithmetic, one rounding).
 * Strides are in elements: token strides of query/key, and the stride between heads.
 * A token whose position is outside [0, max_position) is left untouched (MCOP_DEVERR_POSITION). */
int mcop_rope_inplace(const int64_t* positions, void* query, void* key, const void* cos_sin_cache,
                      int cache_dtype, int64_t max_position, int64_t tokens, int num_heads, int num_kv_heads,
                      int head_size, int rot_dim, int64_t query_stride, int64_t key_stride, int64_t head_stride,
                      int is_neox, int dtype, mcop_stream_t stream);

/* mcoplib.op.rotary_embedding, op/rotary_embedding.cu:99-121 (include/rotary_embedding.h:3-5).
 * NeoX RoPE of the Q and K heads of packed_qkv [tokens, Hq+2Hkv, D] into output (same layout, V heads not
 * touched); position of token t of sequence b = cache_lens[b] + t - accum_q_lens[b];
 * cos, sin fp32 [max_position, D/2]; fp32 arithmetic, one rounding.  A token whose position is outside
 * [0, max_position) is not written (MCOP_DEVERR_POSITION). */
int mcop_rope_packed(const void* packed_qkv, void* output, const float* cos, const float* sin, int64_t max_position,
                     const int32_t* accum_q_lens, const int32_t* cache_lens, int batch, int64_t tokens,
                     int q_heads, int kv_heads, int head_dim, int dtype, mcop_stream_t stream);

/* mcoplib.op.fused_rope_fwd, op/fused_rope.cu:13-74 (kernel/fused_rope_kernel.h:6-96).
 * In-place NeoX RoPE of the Q and K planes of qkv [seq, planes>=2, heads, D]; cos, sin [max_position, D/2] in the
 * activation dtype; row = indexes[s] (int64) or s when indexes is NULL; fp32 arithmetic, one rounding.
 * A row outside [0, max_position) leaves its token untouched (MCOP_DEVERR_POSITION).
 * out_bf16 != 0 (the reference's force_bf16_attn, f16 data only, :44-52): the rotated Q and K heads are rounded to and
 * stored as bf16 in place of the f16 values; the other planes keep their f16 bits, as in the reference. */
int mcop_fused_rope_fwd(void* qkv, const void* cos, const void* sin, int64_t max_position, const int64_t* indexes,
                        int64_t seq, int planes, int heads, int head_dim, int dtype, int out_bf16, mcop_stream_t stream);

/* mcoplib.op.fused_rope_bwd, op/fused_rope.cu:77-138 (kernel/fused_rope_kernel.h:101-191).
 * The transposed rotation (gradient of fused_rope_fwd), same layout and arguments:
 * x' = x*c + y*s, y' = y*c - x*s in fp32, one rounding. */
int mcop_fused_rope_bwd(void* qkv, const void* cos, const void* sin, int64_t max_position, const int64_t* indexes,
                        int64_t seq, int planes, int heads, int head_dim, int dtype, int out_bf16, mcop_stream_t stream);

/* mcoplib.op.store_kv_cache_cuda_interface, op/store_kv.cu:220-350 (include/store_kv.h:2-15).
 * code = clamp(rne(x * scale[h, d]), -127, 127) for the K and V heads of packed_qkv
 * (strides qkv_stride_token / qkv_stride_head, elements) written to cache[slot_ids[b], h, cache_lens[b] + i, :]
 * with cache strides in bytes-as-elements (int8): stride_slot, stride_head, stride_pos.  The caches hold num_slots
 * slots of max_len positions; a token whose slot id or position falls outside is not stored (MCOP_DEVERR_KV_INDEX). */
int mcop_kv_store_i8(const void* packed_qkv, int64_t qkv_stride_token, int64_t qkv_stride_head,
                     const int32_t* q_lens, const int32_t* accum_q_lens, const int32_t* cache_lens,
                     const int32_t* cache_slot_ids, int8_t* k_cache, int8_t* v_cache, int64_t num_slots, int64_t max_len,
                     int64_t k_stride_slot, int64_t k_stride_head, int64_t k_stride_pos,
                     int64_t v_stride_slot, int64_t v_stride_head, int64_t v_stride_pos,
                     const float* k_scale, const float* v_scale, int batch, int64_t tokens, int q_heads,
                     int kv_heads, int head_dim, int dtype, mcop_stream_t stream);

/* torch.ops._C_cache_ops.reshape_and_cache_flash with kv_cache_dtype "auto",
 * op/vllm/cache_kernels.cu:193-266,610-650 (schema torch_bindings.cpp:412-420).
 * Copies key/value [tokens, kv_heads, head_size] (token stride given) to the paged cache at
 * slot_mapping[t] (block = slot / block_size, offset = slot % block_size; negative = skip).
 * The cache is addressed by strides (elements): block, in-block position, head; head_size contiguous.
 * A slot >= num_blocks * block_size is skipped (MCOP_DEVERR_SLOT). */
int mcop_reshape_and_cache_flash(const void* key, const void* value, int64_t key_stride, int64_t value_stride,
                                 void* key_cache, void* value_cache, int64_t block_stride, int64_t page_stride,
                                 int64_t head_stride, const int64_t* slot_mapping, int64_t tokens,
                                 int kv_heads, int head_size, int block_size, int64_t num_blocks, int elem_bytes,
                                 mcop_stream_t stream);

/* torch.ops._C_cache_ops.reshape_and_cache with kv_cache_dtype "auto",
 * op/vllm/cache_kernels.cu:133-190,564-593 (schema torch_bindings.cpp:403-409): the split layout of the paged cache,
 * key_cache [num_blocks, kv_heads, head_size / x, block_size, x] and value_cache [num_blocks, kv_heads, head_size,
 * block_size], both contiguous.  key/value [tokens, kv_heads, head_size] with token strides in elements;
 * block = slot / block_size, offset = slot % block_size; a negative slot is skipped, a slot >= num_blocks * block_size
 * is skipped and reported (MCOP_DEVERR_SLOT).  head_size % x == 0.  Every (head, group of x) is copied - the reference
 * launches at most 512 threads per token and leaves the groups beyond them unwritten (:575). */
int mcop_reshape_and_cache(const void* key, const void* value, int64_t key_stride, int64_t value_stride,
                           void* key_cache, void* value_cache, const int64_t* slot_mapping, int64_t tokens,
                           int kv_heads, int head_size, int block_size, int x, int64_t num_blocks, int elem_bytes,
                           mcop_stream_t stream);

/* sglang's apply_rope_pos_ids_cos_sin_cache with save_kv_cache (op/sglang/csrc/elementwise/rope.cu:28-171, the kernel it
 * calls fuses rotation and save): NeoX RoPE over the whole head from an fp32 cos||sin cache [max_position, head_size] at
 * explicit positions, query and key rotated in place (fp32 products and sum, one rounding), then
 * k_buffer[kv_loc[t]] = rotated key row, v_buffer[kv_loc[t]] = value row, in the element type; the buffers hold
 * buffer_rows rows of kv_heads * head_size elements, buffer_row_stride elements apart.  One launch from 2048 tokens on
 * 16-byte aligned rows; otherwise the rotation followed by the copy.  Positions and row ids are checked like those of
 * mcop_rope_kv_store_i8_paged (MCOP_DEVERR_POSITION / MCOP_DEVERR_SLOT; a negative row id rotates and does not store). */
int mcop_rope_kv_copy(const int64_t* positions, void* query, void* key, const void* value, const float* cos_sin_cache,
                      int64_t max_position, void* k_buffer, void* v_buffer, const int64_t* kv_loc, int64_t buffer_rows,
                      int64_t buffer_row_stride, int64_t tokens, int num_heads, int num_kv_heads, int head_size,
                      int64_t query_stride, int64_t key_stride, int64_t value_stride, int dtype, mcop_stream_t stream);

/* Fused RoPE + int8 paged KV store.  No single reference operator: the composition of
 * rotary_embedding (op/vllm/pos_encoding_kernels.cu:135-217) -> int8 quantisation of the ROUNDED rotated K
 * and of V as in op/store_kv.cu:188-216 with per-head dequantisation scales (code = clamp(rne(v * (1/scale[h])), +-127))
 * -> paged addressing of op/vllm/cache_kernels.cu:204-222.  query and key are rotated in place.
 * key_cache/value_cache int8 [num_blocks, block_size, kv_heads, head_size] contiguous;
 * k_scale, v_scale fp32 [kv_heads].  A token whose position is outside [0, max_position) is left untouched and not
 * stored (MCOP_DEVERR_POSITION); a slot >= num_blocks * block_size is rotated but not stored (MCOP_DEVERR_SLOT);
 * a negative slot is rotated and not stored (the caller's "no store" mark, not an error). */
int mcop_rope_kv_store_i8_paged(const int64_t* positions, void* query, void* key, const void* value,
                                const void* cos_sin_cache, int cache_dtype, int64_t max_position, int8_t* key_cache,
                                int8_t* value_cache, const int64_t* slot_mapping, const float* k_scale,
                                const float* v_scale, int64_t tokens, int num_heads, int num_kv_heads,
                                int head_size, int rot_dim, int64_t query_stride, int64_t key_stride,
                                int64_t value_stride, int block_size, int64_t num_blocks, int is_neox,
                                int dtype, mcop_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Part 3 - MoE routing, dispatch (scatter + quant) and combine (gather)
 * ---------------------------------------------------------------------------------------------- */

/* mcoplib.op.moe_softmax_topk, op/moe_softmax_topk.cu:216-235 (include/moe_softmax_topk.h:3-7).
 * fp32 logits [tokens, experts] -> softmax -> top-k (ties to the lowest index, descending order) ->
 * weights renormalised to sum 1.  experts <= 1024, 1 <= k <= min(experts, 32). */
int mcop_moe_softmax_topk(float* topk_weights, int32_t* topk_ids, const float* logits, int64_t tokens,
                          int experts, int k, mcop_stream_t stream);

/* torch.ops._moe_C.topk_softmax, op/vllm/moe/topk_softmax_kernels.cu:884-918 (schema op/vllm/moe/torch_bindings.cpp:6-9):
 * logits [tokens, experts] in fp32 / bf16 / f16 -> fp32 softmax -> top-k (ties to the lowest index, descending order);
 * the weights are the softmax probabilities, divided by their sum only when renormalize != 0.
 * token_expert_indices (nullable) int32 [tokens, k] receives j * tokens + t.  experts <= 1024, k <= min(experts, 32). */
int mcop_topk_softmax(float* topk_weights, int32_t* topk_ids, int32_t* token_expert_indices, const void* logits,
                      int64_t tokens, int experts, int k, int renormalize, int logits_dtype, mcop_stream_t stream);

/* mcoplib.op.fused_moe_gate_deepseek, op/fused_moe_gate_deepseek.cu:63-138 (include/fused_moe_gate_deepseek.h:6-18;
 * kernels kernel/fused_moe_gate_deepseek.cuh:129-243,316-374).  Sigmoid scores + bias, group score = two best biased
 * scores, keep topk_group groups, top-k experts of the kept groups (ties to the lower index, descending biased score).
 * moegate_type 0 (DEEPSEEK): weights = score / sum(selected scores) (if renormalize) * routed_scaling; no shared experts.
 * moegate_type 1 (SGLANG): tot = fp32 sum of the routed scores; weights = T(score / T(tot)) if renormalize, else the
 *   score; never scaled.  With num_fused_shared_experts == 1 the last of the topk slots is the fused shared expert:
 *   id = experts, weight = T(T(tot) * T(1 / routed_scaling)), divided by T(tot) like the others when renormalize; topk - 1
 *   routed experts are selected.  num_fused_shared_experts > 1 is rejected (the reference draws those ids from the clock).
 * experts % 32 == 0, experts <= 512; groups == 1, or experts/groups a multiple of experts/32 spanning a
 * power-of-two number of lanes.  group_mask (nullable) int32 [tokens]: bit g set iff group g was kept. */
int mcop_moe_gate_grouped_sigmoid(const void* logits, const void* bias, float* topk_weights,
                                  int32_t* topk_ids, int32_t* group_mask, int64_t tokens, int experts,
                                  int groups, int topk_group, int topk, int renormalize,
                                  float routed_scaling, int num_fused_shared_experts, int moegate_type,
                                  int logits_dtype, int bias_dtype, mcop_stream_t stream);

/* mcoplib.op.fused_moe_gate_opt, op/moe_fused_gate_opt.cu:9-92 (kernels kernel/fused_moe_gate.cuh:137-251,346-463):
 * the same selection as mcop_moe_gate_grouped_sigmoid with logits and bias of one dtype, and sglang's weights:
 * routed weight = T(score / T(fp32 sum of the selected scores)) when renormalize, else the score; never scaled.
 * With num_shared_experts == 1 the last of the topk slots is the fused shared expert: id = experts, weight =
 * (sum of the routed weights) / routed_scaling when renormalize, else 0; topk - 1 routed experts are selected.
 * num_shared_experts > 1 is rejected (the reference fills those ids from rand()). */
int mcop_moe_gate_grouped_sigmoid_shared(const void* logits, const void* bias, float* topk_weights,
                                         int32_t* topk_ids, int64_t tokens, int experts, int groups,
                                         int topk_group, int topk, int renormalize, int num_shared_experts,
                                         double routed_scaling, int dtype, mcop_stream_t stream);

/* torch.ops._moe_C.grouped_topk, op/vllm/moe/grouped_topk_kernels.cu:962-1060 (kernels :560-870; schema
 * op/vllm/moe/torch_bindings.cpp:86-91): score = x (scoring_func 0) or T(0.5 * tanh(0.5 x) + 0.5) (scoring_func 1);
 * biased = T(score + bias); group score = T(best + second best biased score of the group); keep topk_group groups, then
 * the top-k experts of the kept groups (ties to the lower index, descending biased score);
 * value = score * (routed_scaling / (1e-20 + sum of the selected scores)) when renormalize, else score * routed_scaling.
 * A token whose topk_group-th group score is -inf or not finite gets ids 0..k-1 and values 1/k, as in the reference.
 * Same shape limits as mcop_moe_gate_grouped_sigmoid; bias dtype = scores dtype or fp32. */
int mcop_grouped_topk(const void* scores, const void* bias, float* topk_values, int32_t* topk_ids, int64_t tokens,
                      int experts, int n_group, int topk_group, int topk, int renormalize, double routed_scaling,
                      int scoring_func, int scores_dtype, int bias_dtype, mcop_stream_t stream);

/* Bytes of scratch mcop_moe_scatter_quant_i8 needs (contents need no initialisation). */
size_t mcop_moe_scatter_workspace_bytes(int64_t tokens, int topk, int experts_per_rank);

/* mcoplib.op.moe_scatter_dynamic_quant with no shared experts, op/moe_scatter_dynamic_quant.cu:312-341
 * (include/moe_scatter_dynamic_quant.h:3-5).  Rows ordered by (expert, token); ids outside
 * [0, experts_per_rank) are dropped.  row = int8(rne(x[t] * w[t,j] * smooth[e] * (127 / absmax))),
 * row_scales = absmax / 127.  hidden bf16 [tokens, hidden]; ids int32 / weights fp32 [tokens, topk];
 * smooth fp32 [experts_per_rank, hidden]; rows int8 [tokens*topk, hidden]; row_scales fp32 and row2tok
 * int32 [tokens*topk]; counts, starts int32 [experts_per_rank]; tok2row (nullable) int32 [tokens, topk]
 * receives the row of every (token, slot), -1 if dropped.  Entries of rows / row_scales / row2tok past the
 * last routed row are left as they are. */
int mcop_moe_scatter_quant_i8(const void* hidden, const int32_t* ids, const float* weights,
                              const float* smooth, int8_t* rows, float* row_scales, int32_t* row2tok,
                              int32_t* counts, int32_t* starts, int32_t* tok2row, int64_t tokens,
                              int64_t hidden_size, int topk, int experts_per_rank, void* workspace,
                              size_t workspace_bytes, mcop_stream_t stream);

/* Bytes of scratch the gathers need when tok2row is NULL (0 otherwise). */
size_t mcop_moe_gather_workspace_bytes(int64_t tokens, int64_t rows);

/* mcoplib.op.moe_gather, op/moe_gather.cu:137-150 (include/moe_gather.h:3-6): out[row2tok[r]] += y[r].
 * Deterministic: acc = float(out[t]); acc += y[r] for the rows of t in ascending r; out[t] = bf16(acc).
 * y bf16 [rows, hidden], out bf16 [tokens, hidden].  tok2row (nullable) int32 [tokens, topk] as written by
 * mcop_moe_scatter_quant_i8 avoids the inversion pre-pass (then workspace may be NULL). */
int mcop_moe_gather(const void* y, const int32_t* row2tok, void* out, const int32_t* tok2row, int topk,
                    int64_t tokens, int64_t rows, int64_t hidden_size, void* workspace,
                    size_t workspace_bytes, mcop_stream_t stream);

/* Weighted combine (no reference counterpart; weight lookup as op/moe_scatter_dynamic_quant.cu:240-247):
 * out[t] = bf16((accumulate ? float(out[t]) : 0) + sum over the rows r of t, ascending, of w[t, j(r)] * y[r]),
 * j(r) = first slot of t whose id equals the expert owning row r (from starts). */
int mcop_moe_gather_weighted(const void* y, const int32_t* row2tok, const int32_t* topk_ids,
                             const float* topk_weights, const int32_t* starts, void* out,
                             const int32_t* tok2row, int accumulate, int64_t tokens, int64_t rows,
                             int64_t hidden_size, int topk, int experts, void* workspace,
                             size_t workspace_bytes, mcop_stream_t stream);

/* mcoplib.op.moe_swiglu_dynamic_quantize, op/moe_swiglu_dq.cu:63-292 (include/moe_swiglu_dq.h): the rows produced by
 * the expert up-projection, x bf16 [rows, 2*hidden] = gate || up, grouped by expert (rows of expert e are
 * [starts[e], starts[e] + counts[e])): v = up * (gate / (1 + exp(-gate))) * smooth[e]; scales = max|v| * (1/127);
 * out = int8(rne(v * (127 / max|v|))) clamped to +-127.  Rows owned by no expert are not written. */
int mcop_moe_swiglu_quant_i8(const void* x, const float* smooth, const int32_t* starts, const int32_t* counts,
                             int8_t* out, float* scales, int64_t rows, int64_t hidden, int experts,
                             mcop_stream_t stream);

/* sglang flavour of the same operator with one more output, rms_norm_dynamic_per_token_quant_custom(out, out_bf16, input,
 * weight, scales, eps, scale_ub, residual): op/sglang/include/sgl_kernel_ops.h:138-145, op/sglang/csrc/common_extension.cc:84-86,
 * op/sglang/csrc/elementwise/fused_layernorm_dynamic_per_token_quant_custom.cu:434-460.  Identical to
 * mcop_add_rmsnorm_quant_i8, and out_norm [tokens, hidden] in T receives n (the normalised row before quantisation). */
int mcop_add_rmsnorm_quant_i8_norm_out(int8_t* out, void* out_norm, float* scales, const void* x, int64_t x_row_stride,
                                       const void* weight, void* residual, const float* scale_ub, int64_t tokens,
                                       int64_t hidden, float eps, int dtype, mcop_stream_t stream);

/* mcoplib.op.fused_add_rms_norm_dynamic_per_token_quant_padding_output,
 * op/fused_add_layernorm_per_token_quant_padding_output.cu:397-416 (include/fused_add_layernorm_per_token_quant_padding_output.h:3-11;
 * wrapper mcoplib/custom_ops.py:7-27): residual add + RMSNorm + per-token int8 quantisation whose primary output is one
 * byte record per token of pad_size_elems 16-bit elements: bytes [0, hidden) the codes, bytes [hidden, hidden+4) the
 * fp32 scale, the rest not written.  residual is updated in place to T(x + residual).  out_norm (T [tokens, hidden]),
 * out_codes (int8 [tokens, hidden]) and out_scales (fp32 [tokens]) are optional (NULL = not wanted).
 * form: 0 = the reference's choice (1 iff hidden == 7168), 1 = its fp32 form (kernel :182-283), 2 = its rounded form
 * (kernel :287-340); the two differ in where values are rounded to T, see the kernel file.  hidden % 4 == 0. */
int mcop_add_rmsnorm_quant_i8_padded(const void* x, void* residual, const void* weight, void* out_packed,
                                     void* out_norm, int8_t* out_codes, float* out_scales, int64_t tokens,
                                     int64_t hidden, int64_t pad_size_elems, float eps, int form, int dtype,
                                     mcop_stream_t stream);

/* mcoplib.op.fused_silu_mul_dq_reorder_quant,op/int8_quant_kernels.cu:1355-1417,1893-1940 (include/int8_quant_kernel.h:7-14),
 * and with row_ids == NULL the unmasked form fused_silu_mul_dq_quant_interface (:1877-1891):
 * x [rows, 2n] = gate || up in dtype (MCOP_BF16 / MCOP_F16); row r is processed iff id_lo <= row_ids[r] <= id_hi
 * (ids int32, or int64 when ids_are_i64), other rows are not written.  v = up * (gate * (1 / (1 + exp(-gate)))) in
 * fp32; scales[r] = max|v| * (1/127); out[r, :] = int8(rne(v * (127 / max|v|))).  The reference accepts a w2_scale
 * tensor and never applies it (both instantiations pass HAS_SCALE = false), so there is no such argument here. */
int mcop_silu_mul_quant_i8(const void* x, int dtype, const void* row_ids, int ids_are_i64, int64_t id_lo,
                           int64_t id_hi, int8_t* out, float* scales, int64_t rows, int64_t n,
                           mcop_stream_t stream);

/* mcoplib.op.fused_silu_mul_dq_mask_quant, op/int8_quant_kernels.cu:881-955,1844-1875 (include/int8_quant_kernel.h:2-5):
 * x [groups, rows_per_group, 2n]; group_counts[g] (int32 / int64) = number of valid rows of group g.  Every valid row
 * becomes one byte record of out_stride_elems * 2 bytes in out_packed [groups, rows_per_group, out_stride_elems]
 * (16-bit elements): bytes [0, n) the int8 codes, bytes [n, n+4) the fp32 scale; other rows and bytes are not
 * written.  Same arithmetic as mcop_silu_mul_quant_i8.  n must be a multiple of 4 (the reference needs 8). */
int mcop_silu_mul_quant_i8_masked_pack(const void* x, int dtype, const void* group_counts, int counts_are_i64,
                                       void* out_packed, int64_t groups, int64_t rows_per_group, int64_t n,
                                       int64_t out_stride_elems, mcop_stream_t stream);

/* Size of the built-in scratch area of mcop_moe_gather_noalloc (bytes held by every GPU that loads the library). */
#define MCOP_GATHER_NOALLOC_SCRATCH_BYTES (4u << 20)

/* mcop_moe_gather for callers that have no way to hand over scratch memory.  No counterpart in the reference.
 *
 * Same result as mcop_moe_gather(y, row2tok, out, tok2row = NULL, ...): out[row2tok[r]] += y[r], rows of a token
 * summed in ascending r in fp32, one bf16 rounding.  The row -> token map is inverted into a scratch table; here
 * that table lives in a fixed MCOP_GATHER_NOALLOC_SCRATCH_BYTES array inside the library instead of a caller
 * workspace, so the call performs no device allocation of any kind (no cudaMalloc / cudaFree, no allocating
 * library routine, no framework allocator).  It is meant for hosts that own nothing but the input and output
 * buffers they were given - a plugin loaded into a serving engine that has already reserved the device memory
 * for its own pool, a bare C host without an allocator, a latency-critical loop where the implicit device
 * synchronisation of an allocation is not acceptable.
 *
 * Limit: mcop_moe_gather_workspace_bytes(tokens, rows) must not exceed MCOP_GATHER_NOALLOC_SCRATCH_BYTES
 * (e.g. 65536 tokens x 8 rows each); larger problems are rejected with MCOP_ERR_WORKSPACE and nothing runs.
 * The first call on a device resolves the device address of the array (cudaGetSymbolAddress with that device
 * current); make that first call outside any stream capture.  All calls on a device share the one array and it
 * keeps the previous call's contents: every call resets the chain heads it needs, but two calls whose kernels
 * overlap on the GPU (different streams, no ordering between them) race on it - serialise them. */
int mcop_moe_gather_noalloc(const void* y, const int32_t* row2tok, void* out, int64_t tokens, int64_t rows,
                            int64_t hidden_size, mcop_stream_t stream);

/* torch.ops._moe_C.moe_sum, op/vllm/moe/moe_align_sum_kernels.cu:352-367,770-815 (schema op/vllm/moe/torch_bindings.cpp:13):
 * output[t, :] = sum_k input[t, k, :], input [tokens, topk, hidden] contiguous, output [tokens, hidden], bf16 / f16 / f32.
 * topk 2, 3, 4: the running sum is kept in the element type (slots in order, every partial sum rounded), as the
 * reference's kernels do; any other topk: fp32 accumulation in slot order, one rounding (the reference calls the
 * framework's reduction there). */
int mcop_moe_sum(const void* input, void* output, int64_t tokens, int topk, int64_t hidden_size, int dtype,
                 mcop_stream_t stream);

/* sglang's moe_sum_reduce, op/sglang/csrc/moe/moe_sum_reduce.cu:119-223,226-330 (schema op/sglang/csrc/common_extension.cc:252):
 * output[t, :] = T((sum_k float(input[t, k, :])) * float(routed_scaling_factor)) - fp32 accumulation in slot order for
 * every topk, one rounding.  Same layouts and types as mcop_moe_sum. */
int mcop_moe_sum_reduce(const void* input, void* output, int64_t tokens, int topk, int64_t hidden_size,
                        double routed_scaling_factor, int dtype, mcop_stream_t stream);

/* torch.ops._moe_C.moe_align_block_size, op/vllm/moe/moe_align_sum_kernels.cu:86-180,612-735
 * (schema op/vllm/moe/torch_bindings.cpp:18-24).  Index preparation of a block-sparse expert GEMM:
 *   sorted_token_ids [max_num_tokens_padded]: for every expert e in ascending order, the flat indices i = t*topk + j
 *     of the routing entries with (mapped) expert e, then the mark `numel` up to a multiple of block_size; every
 *     position after the last expert's range also holds `numel`;
 *   expert_ids [max_num_blocks]: the expert of every block of block_size positions; blocks after the padded total: 0;
 *   num_tokens_post_pad [1]: the padded total.
 * Entries with id outside [0, num_experts) are dropped; with expert_map (int32 [num_experts], NULL = identity) the id
 * is mapped first and entries mapped to -1 are dropped.  Inside an expert's range the reference's order depends on
 * its atomics; here it is ascending flat index (one of the orders the reference can produce; its own check sorts the
 * ranges before comparing).  num_experts < 1024.  Scratch: mcop_moe_align_block_size_workspace_bytes(). */
size_t mcop_moe_align_block_size_workspace_bytes(int64_t numel, int num_experts);
int mcop_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int num_experts, int block_size,
                              int32_t* sorted_token_ids, int64_t max_num_tokens_padded, int32_t* expert_ids,
                              int64_t max_num_blocks, int32_t* num_tokens_post_pad, const int32_t* expert_map,
                              void* workspace, size_t workspace_bytes, mcop_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MCOP_B200_H_ */
