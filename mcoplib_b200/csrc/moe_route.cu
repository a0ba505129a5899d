// Part 3a of the hot path: MoE routers.
//
// Both routers keep a token's expert scores in registers and do every reduction (row max, row sum,
// group top-2, group selection, the k rounds of arg-max) with warp shuffles: no shared memory, no block
// barrier.  Ties always go to the lower index.
#include <math.h>

#include "common.cuh"
#include "tma_pipe.cuh"

namespace mcop {
namespace {

__device__ __forceinline__ bool better(float v, int i, float ov, int oi) {
  // true if (ov, oi) beats (v, i): larger value, or equal value and lower index
  return ov > v || (ov == v && oi < i);
}

// Order-preserving map from float to unsigned (a < b  <=>  key(a) < key(b) for non-NaN values), so that warp-wide
// integer max (redux.sync) can stand in for a float max.
__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// ---------------------------------------------------------------------------------------------
// softmax + top-k.  A row is spread over TPR lanes (a power of two), VPT contiguous experts per lane.
// ---------------------------------------------------------------------------------------------
// LT: logits type.  renorm: divide the k weights by their sum.  src_rows (nullable): vLLM's token_expert_indices,
// src_rows[t, j] = j * tokens + t.
template <typename LT, int VPT, int TPR>
__global__ void __launch_bounds__(128) softmax_topk_kernel(float* __restrict__ weights, int32_t* __restrict__ ids,
                                                           int32_t* __restrict__ src_rows, const LT* __restrict__ logits,
                                                           int64_t tokens, int experts, int k, bool vec_ok, bool renorm) {
  constexpr int ROWS_PER_WARP = 32 / TPR;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int g = lane % TPR;
  const int64_t row = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * ROWS_PER_WARP + lane / TPR;
  const bool active = row < tokens;
  const int first = g * VPT;
  float p[VPT];
  if (sizeof(LT) == 4 && active && vec_ok) {
    const float4* src = reinterpret_cast<const float4*>(logits + row * experts + first);
#pragma unroll
    for (int i = 0; i < VPT / 4; ++i) {
      const float4 v = __ldg(src + i);
      p[4 * i] = v.x; p[4 * i + 1] = v.y; p[4 * i + 2] = v.z; p[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      p[i] = (active && first + i < experts) ? ElemTraits<LT>::to_float(logits[row * experts + first + i]) : -INFINITY;
  }
  float m = p[0];
#pragma unroll
  for (int i = 1; i < VPT; ++i) m = fmaxf(m, p[i]);
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    p[i] = expf(p[i] - m);
    sum += p[i];
  }
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float rcp = 1.0f / sum;
#pragma unroll
  for (int i = 0; i < VPT; ++i) p[i] = p[i] * rcp;

  float tot = 0.f;
  for (int kk = 0; kk < k; ++kk) {
    float bv = p[0];
    int bi = first;
#pragma unroll
    for (int i = 1; i < VPT; ++i)
      if (p[i] > bv) { bv = p[i]; bi = first + i; }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(bv, bi, ov, oi)) { bv = ov; bi = oi; }
    }
    if (active && g == 0) {
      weights[row * k + kk] = bv;
      ids[row * k + kk] = bi;
      if (src_rows) src_rows[row * k + kk] = (int32_t)(kk * tokens + row);
      tot += bv;
    }
    if (bi / VPT == g) {
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        if (i == bi % VPT) p[i] = -1.0f;  // probabilities are >= 0
    }
  }
  if (renorm && active && g == 0) {
    const float denom = tot > 0.f ? tot : 1.f;
    for (int kk = 0; kk < k; ++kk) weights[row * k + kk] = weights[row * k + kk] / denom;
  }
}

template <typename LT, int VPT, int TPR>
int launch_softmax(float* w, int32_t* ids, int32_t* src_rows, const LT* logits, int64_t tokens, int experts, int k, bool renorm,
                   cudaStream_t s) {
  constexpr int WARPS = 4;
  const int64_t rows_per_block = WARPS * (32 / TPR);
  const int64_t blocks = (tokens + rows_per_block - 1) / rows_per_block;
  MCOP_REQUIRE(blocks <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "moe_softmax_topk: too many tokens");
  const bool vec_ok = experts == VPT * TPR && aligned16(logits);
  (void)launch_pdl(softmax_topk_kernel<LT, VPT, TPR>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, s, w, ids, src_rows, logits, tokens, experts, k,
                   vec_ok, renorm);
  return check_launch("moe_softmax_topk");
}

template <typename LT>
int dispatch_softmax(float* w, int32_t* ids, int32_t* src_rows, const LT* logits, int64_t tokens, int experts, int k, bool renorm,
                     cudaStream_t s) {
  if (experts <= 8) return launch_softmax<LT, 8, 1>(w, ids, src_rows, logits, tokens, experts, k, renorm, s);
  if (experts <= 16) return launch_softmax<LT, 8, 2>(w, ids, src_rows, logits, tokens, experts, k, renorm, s);
  if (experts <= 32) return launch_softmax<LT, 8, 4>(w, ids, src_rows, logits, tokens, experts, k, renorm, s);
  if (experts <= 64) return launch_softmax<LT, 8, 8>(w, ids, src_rows, logits, tokens, experts, k, renorm, s);
  if (experts <= 128) return launch_softmax<LT, 8, 16>(w, ids, src_rows, logits, tokens, experts, k, renorm, s);
  if (experts <= 256) return launch_softmax<LT, 8, 32>(w, ids, src_rows, logits, tokens, experts, k, renorm, s);
  if (experts <= 512) return launch_softmax<LT, 16, 32>(w, ids, src_rows, logits, tokens, experts, k, renorm, s);
  return launch_softmax<LT, 32, 32>(w, ids, src_rows, logits, tokens, experts, k, renorm, s);
}

// ---------------------------------------------------------------------------------------------
// Grouped sigmoid gate.  One warp per token, V = experts / 32 contiguous experts per lane, so a group of
// experts/groups experts is a run of adjacent lanes.
// ---------------------------------------------------------------------------------------------
struct GateParams {
  const void* logits; const void* bias; float* weights; int32_t* ids; int32_t* group_mask;
  int64_t tokens; int experts, groups, topk_group, topk, renormalize; float scaling;
  int t1, ts;  // dtype codes: logits type, and the wider of logits/bias types
  // style 0: mcoplib.op.fused_moe_gate_deepseek weights.  style 1: mcoplib.op.fused_moe_gate_opt weights
  // (kernel/fused_moe_gate.cuh:346-420): the last `shared` of the topk slots name the fused shared expert
  // (id = experts) instead of a routed expert; routed weights are not scaled.
  // style 2: torch.ops._moe_C.grouped_topk (op/vllm/moe/grouped_topk_kernels.cu:560-870): score = x (scoring 0) or
  // T(0.5 * tanh(0.5 x) + 0.5) (scoring 1); biased = T(score + float(bias)); non-finite logits never win an expert slot,
  // non-finite group scores count as -inf, and a token whose topk_group-th group score is -inf gets ids 0..k-1 with
  // weights 1/k; weight = score * (scaling / (1e-20 + fp32 butterfly sum of the selected scores)) when renormalize.
  // style 3: mcoplib.op.fused_moe_gate_deepseek with moegate_type 1 (kernel/fused_moe_gate_deepseek.cuh:334-374):
  // tot = fp32 16-lane butterfly sum of the routed scores; the shared slot (if any) gets id = experts and
  // T(T(tot) * T(scaling)); with renormalize every slot becomes T(T(w) / T(tot)); routed weights are not scaled
  // (`scaling` holds 1 / routed_scaling_factor, as the reference's host code computes it).
  int style, shared;
  double shared_mul;  // style 1: weight of the shared slot = sum of the routed weights * shared_mul
  int scoring;        // style 2 only
  int vec_ok;         // the logits rows are 16-byte aligned: fp32 logits may be read as float4
};

template <typename T1, typename T2, int V>
__global__ void __launch_bounds__(128) gate_kernel(GateParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= p.tokens) return;  // whole warp leaves together
  const int first = lane * V;
  const T1* x = reinterpret_cast<const T1*>(p.logits) + row * p.experts + first;
  const T2* b = reinterpret_cast<const T2*>(p.bias) + first;
  float score[V], biased[V];
  float xin[V];
  if (sizeof(T1) == 4 && V % 4 == 0 && p.vec_ok) {
#pragma unroll
    for (int i = 0; i < V / 4; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
      xin[4 * i] = v.x; xin[4 * i + 1] = v.y; xin[4 * i + 2] = v.z; xin[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) xin[i] = ElemTraits<T1>::to_float(x[i]);
  }
  const bool vllm_form = p.style == 2;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    if (vllm_form) {
      score[i] = p.scoring == 0 ? xin[i] : round_code(0.5f * tanhf(0.5f * xin[i]) + 0.5f, p.t1);
      biased[i] = round_code(score[i] + ElemTraits<T2>::to_float(b[i]), p.t1);
    } else {
      score[i] = round_code(1.0f / (1.0f + expf(-xin[i])), p.t1);
      biased[i] = round_code(score[i] + round_code(ElemTraits<T2>::to_float(b[i]), p.ts), p.ts);
    }
  }

  unsigned sel = 0xffffffffu;
  bool fallback = false;  // style 2: no valid group choice, uniform default routing
  if (p.groups > 1) {
    const int lpg = (p.experts / p.groups) / V;  // lanes per group, a power of two
    float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float v = biased[i];
      if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) m2 = v;
    }
    for (int o = lpg >> 1; o > 0; o >>= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, m1, o);
      const float o2 = __shfl_xor_sync(0xffffffffu, m2, o);
      const float n1 = fmaxf(m1, o1);
      const float n2 = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
      m1 = n1; m2 = n2;
    }
    float gscore = round_code(m1 + m2, p.ts);
    if (vllm_form && !isfinite(gscore)) gscore = -INFINITY;
    const int gid = lane / lpg;
    sel = 0;
    // One warp-wide integer max (redux.sync) on an order-preserving key finds the best remaining group score; the
    // lowest lane holding it belongs to the lowest group index (lanes are ordered by group).
    unsigned best = 0;
    for (int r = 0; r < p.topk_group; ++r) {
      const unsigned key = ((sel >> gid) & 1u) ? 0u : ordered_key(gscore);
      best = __reduce_max_sync(0xffffffffu, key);
      const unsigned who = __ballot_sync(0xffffffffu, key == best);
      const int win = (__ffs(who) - 1) / lpg;
      sel |= 1u << win;
    }
    fallback = vllm_form && best <= ordered_key(-INFINITY);
    if (!((sel >> gid) & 1u)) {
#pragma unroll
      for (int i = 0; i < V; ++i) biased[i] = -INFINITY;
    }
    if (p.group_mask && lane == 0) p.group_mask[row] = (int32_t)sel;
  } else if (p.group_mask && lane == 0) {
    p.group_mask[row] = 1;
  }

  if (vllm_form) {
#pragma unroll
    for (int i = 0; i < V; ++i)
      if (!isfinite(xin[i])) biased[i] = -INFINITY;
  }

  float my_w = 0.f;
  int my_id = 0;
  const int routed = p.topk - p.shared;
  for (int kk = 0; kk < routed; ++kk) {
    // local arg-max (lowest index wins inside the lane), then one redux.sync on the order-preserving key and a
    // ballot: the lowest lane holding the warp maximum owns the lowest expert index among equals
    float bv = biased[0], bs = score[0];
    int bl = 0;
#pragma unroll
    for (int i = 1; i < V; ++i)
      if (biased[i] > bv) { bv = biased[i]; bs = score[i]; bl = i; }
    const unsigned key = ordered_key(bv);
    const unsigned best = __reduce_max_sync(0xffffffffu, key);
    const int src = __ffs(__ballot_sync(0xffffffffu, key == best)) - 1;
    const int bi = __shfl_sync(0xffffffffu, first + bl, src);
    const float sc = __shfl_sync(0xffffffffu, bs, src);
    if (lane == src) {
#pragma unroll
      for (int i = 0; i < V; ++i)
        if (i == bl) biased[i] = -INFINITY;
    }
    if (lane == kk) { my_w = sc; my_id = bi; }
  }
  if (vllm_form) {
    float w;
    if (fallback) {
      my_id = lane;
      w = 1.0f / (float)p.topk;
    } else {
      float sum = lane < p.topk ? my_w : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      float scale = p.scaling;
      if (p.renormalize) scale /= 1e-20f + sum;
      w = my_w * scale;
    }
    if (lane < p.topk) {
      p.weights[row * p.topk + lane] = w;
      p.ids[row * p.topk + lane] = my_id;
    }
    return;
  }
  if (p.style == 3) {
    float tot = lane < routed ? my_w : 0.f;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (p.shared && lane == p.topk - 1) {
      my_id = p.experts;
      my_w = round_code(round_code(tot, p.t1) * round_code(p.scaling, p.t1), p.t1);
    }
    if (p.renormalize) my_w = round_code(round_code(my_w, p.t1) / round_code(tot, p.t1), p.t1);
    if (lane < p.topk) {
      p.weights[row * p.topk + lane] = my_w;
      p.ids[row * p.topk + lane] = my_id;
    }
    return;
  }
  if (p.style == 1) {
    // fp32 sum over a 16-lane xor-butterfly (offsets 8, 4, 2, 1) of the routed scores, one rounding of the sum and
    // one of the quotient to the logits type (kernel/fused_moe_gate.cuh:361-385); lanes >= routed contribute 0
    auto sum16 = [&](float v) {
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      return v;
    };
    const float tot = sum16(lane < routed ? my_w : 0.f);
    if (p.renormalize) my_w = round_code(my_w / round_code(tot, p.t1), p.t1);
    if (p.shared) {
      // the shared slot: id = experts, weight = (sum of the final routed weights) * shared_mul, only when renormalising
      const float tot2 = sum16(lane < routed ? my_w : 0.f);
      if (lane >= routed) {
        my_id = p.experts;
        my_w = p.renormalize ? (float)((double)tot2 * p.shared_mul) : 0.f;
      }
    }
    if (lane < p.topk) {
      p.weights[row * p.topk + lane] = my_w;
      p.ids[row * p.topk + lane] = my_id;
    }
    return;
  }
  if (p.renormalize) {
    float tot;
    if (p.topk == 8) {
      // xor-butterfly over the 8 result lanes, rounding every partial sum to the logits type
      tot = my_w;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) tot = round_code(tot + __shfl_xor_sync(0xffffffffu, tot, o), p.t1);
    } else {
      tot = 0.f;
      for (int j = 0; j < p.topk; ++j) tot = round_code(tot + __shfl_sync(0xffffffffu, my_w, j), p.t1);
    }
    my_w = round_code(my_w / tot, p.t1);
  }
  if (lane < p.topk) {
    p.weights[row * p.topk + lane] = my_w * p.scaling;
    p.ids[row * p.topk + lane] = my_id;
  }
}

template <typename T1, typename T2>
int launch_gate_v(const GateParams& p, cudaStream_t s) {
  constexpr int WARPS = 4;
  const int64_t blocks = (p.tokens + WARPS - 1) / WARPS;
  MCOP_REQUIRE(blocks <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "moe_gate: too many tokens");
  const unsigned gb = (unsigned)blocks;
  switch (p.experts / 32) {
#define MCOP_GATE_CASE(V) case V: (void)launch_pdl(gate_kernel<T1, T2, V>, dim3(gb), dim3(WARPS * 32), 0, s, p); break;
    MCOP_GATE_CASE(1) MCOP_GATE_CASE(2) MCOP_GATE_CASE(3) MCOP_GATE_CASE(4) MCOP_GATE_CASE(5) MCOP_GATE_CASE(6) MCOP_GATE_CASE(8)
    MCOP_GATE_CASE(10) MCOP_GATE_CASE(12) MCOP_GATE_CASE(14) MCOP_GATE_CASE(16)
#undef MCOP_GATE_CASE
    default: return set_error(MCOP_ERR_UNSUPPORTED, "moe_gate: %d experts not supported", p.experts);
  }
  return check_launch("moe_gate");
}

template <typename T1>
int launch_gate_bias(const GateParams& p, int bias_dtype, cudaStream_t s) {
  if (bias_dtype == MCOP_F32) return launch_gate_v<T1, float>(p, s);
  if (bias_dtype == ElemTraits<T1>::code) return launch_gate_v<T1, T1>(p, s);
  return set_error(MCOP_ERR_UNSUPPORTED, "moe_gate: bias dtype must be fp32 or the logits dtype");
}

}  // namespace
}  // namespace mcop

using namespace mcop;

extern "C" int mcop_moe_softmax_topk(float* topk_weights, int32_t* topk_ids, const float* logits, int64_t tokens,
                                     int experts, int k, mcop_stream_t stream) {
  MCOP_REQUIRE(topk_weights && topk_ids && logits, MCOP_ERR_ARGUMENT, "moe_softmax_topk: null pointer");
  MCOP_REQUIRE(tokens >= 0 && experts >= 1 && k >= 1 && k <= experts && k <= 32, MCOP_ERR_ARGUMENT,
               "moe_softmax_topk: bad sizes tokens=%lld experts=%d k=%d", (long long)tokens, experts, k);
  MCOP_REQUIRE(experts <= 1024, MCOP_ERR_UNSUPPORTED, "moe_softmax_topk: more than 1024 experts");
  if (tokens == 0) return MCOP_OK;
  return dispatch_softmax<float>(topk_weights, topk_ids, nullptr, logits, tokens, experts, k, true, (cudaStream_t)stream);
}

extern "C" int mcop_topk_softmax(float* topk_weights, int32_t* topk_ids, int32_t* token_expert_indices, const void* logits,
                                 int64_t tokens, int experts, int k, int renormalize, int logits_dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(topk_weights && topk_ids && logits, MCOP_ERR_ARGUMENT, "topk_softmax: null pointer");
  MCOP_REQUIRE(tokens >= 0 && experts >= 1 && k >= 1 && k <= experts && k <= 32, MCOP_ERR_ARGUMENT,
               "topk_softmax: bad sizes tokens=%lld experts=%d k=%d", (long long)tokens, experts, k);
  MCOP_REQUIRE(experts <= 1024, MCOP_ERR_UNSUPPORTED, "topk_softmax: more than 1024 experts");
  MCOP_REQUIRE(!token_expert_indices || tokens * k <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "topk_softmax: tokens*k exceeds int32");
  if (tokens == 0) return MCOP_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const bool rn = renormalize != 0;
  switch (logits_dtype) {
    case MCOP_F32: return dispatch_softmax<float>(topk_weights, topk_ids, token_expert_indices, reinterpret_cast<const float*>(logits), tokens, experts, k, rn, s);
    case MCOP_BF16: return dispatch_softmax<__nv_bfloat16>(topk_weights, topk_ids, token_expert_indices, reinterpret_cast<const __nv_bfloat16*>(logits), tokens, experts, k, rn, s);
    case MCOP_F16: return dispatch_softmax<__half>(topk_weights, topk_ids, token_expert_indices, reinterpret_cast<const __half*>(logits), tokens, experts, k, rn, s);
  }
  return set_error(MCOP_ERR_UNSUPPORTED, "topk_softmax: unknown logits dtype %d", logits_dtype);
}

static int gate_entry(const void* logits, const void* bias, float* topk_weights, int32_t* topk_ids, int32_t* group_mask,
                      int64_t tokens, int experts, int groups, int topk_group, int topk_total, int renormalize,
                      float routed_scaling, int logits_dtype, int bias_dtype, int style, int shared, double shared_mul,
                      int scoring, mcop_stream_t stream) {
  MCOP_REQUIRE(logits && bias && topk_weights && topk_ids, MCOP_ERR_ARGUMENT, "moe_gate: null pointer");
  MCOP_REQUIRE(shared >= 0 && shared <= 1 && topk_total - shared >= 1, MCOP_ERR_UNSUPPORTED,
               "moe_gate: %d fused shared experts (0 or 1 supported: the reference draws the ids of more from rand())", shared);
  MCOP_REQUIRE((style != 1 && style != 3) || topk_total <= 16, MCOP_ERR_UNSUPPORTED, "moe_gate: at most 16 slots in this form");
  const int topk = topk_total - shared;  // routed experts to select
  MCOP_REQUIRE(tokens >= 0 && experts > 0 && topk >= 1 && topk_total <= 32, MCOP_ERR_ARGUMENT, "moe_gate: bad sizes");
  MCOP_REQUIRE(experts % 32 == 0 && experts <= 512, MCOP_ERR_UNSUPPORTED,
               "moe_gate: experts must be a multiple of 32 and at most 512 (got %d)", experts);
  if (groups < 1) groups = 1;
  const int V = experts / 32;
  if (groups > 1) {
    MCOP_REQUIRE(experts % groups == 0 && groups <= 32, MCOP_ERR_UNSUPPORTED, "moe_gate: %d groups for %d experts", groups, experts);
    const int gs = experts / groups;
    MCOP_REQUIRE(gs % V == 0 && ((gs / V) & (gs / V - 1)) == 0, MCOP_ERR_UNSUPPORTED,
                 "moe_gate: group size %d does not map to a power-of-two number of lanes", gs);
    MCOP_REQUIRE(topk_group >= 1 && topk_group <= groups && (int64_t)topk_group * gs >= topk && gs >= 2, MCOP_ERR_ARGUMENT,
                 "moe_gate: topk_group=%d cannot supply topk=%d", topk_group, topk);
  } else {
    MCOP_REQUIRE(topk <= experts, MCOP_ERR_ARGUMENT, "moe_gate: topk > experts");
  }
  if (tokens == 0) return MCOP_OK;
  GateParams p{logits, bias, topk_weights, topk_ids, group_mask, tokens, experts, groups, topk_group, topk_total,
               renormalize, routed_scaling, logits_dtype, 0, style, shared, shared_mul, scoring, aligned16(logits) ? 1 : 0};
  const int s1 = logits_dtype == MCOP_F32 ? 4 : 2, s2 = bias_dtype == MCOP_F32 ? 4 : 2;
  p.ts = s1 >= s2 ? logits_dtype : bias_dtype;
  cudaStream_t s = (cudaStream_t)stream;
  switch (logits_dtype) {
    case MCOP_F32: return launch_gate_bias<float>(p, bias_dtype, s);
    case MCOP_BF16: return launch_gate_bias<__nv_bfloat16>(p, bias_dtype, s);
    case MCOP_F16: return launch_gate_bias<__half>(p, bias_dtype, s);
  }
  return set_error(MCOP_ERR_UNSUPPORTED, "moe_gate: unknown logits dtype %d", logits_dtype);
}

extern "C" int mcop_moe_gate_grouped_sigmoid(const void* logits, const void* bias, float* topk_weights,
                                             int32_t* topk_ids, int32_t* group_mask, int64_t tokens, int experts,
                                             int groups, int topk_group, int topk, int renormalize,
                                             float routed_scaling, int num_fused_shared_experts, int moegate_type,
                                             int logits_dtype, int bias_dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(moegate_type == 0 || moegate_type == 1, MCOP_ERR_ARGUMENT, "moe_gate: moegate_type must be 0 (DEEPSEEK) or 1 (SGLANG)");
  if (moegate_type == 0) {
    MCOP_REQUIRE(num_fused_shared_experts == 0, MCOP_ERR_UNSUPPORTED,
                 "moe_gate: fused shared experts exist only with moegate_type 1 (as in the reference's dispatch table)");
    return gate_entry(logits, bias, topk_weights, topk_ids, group_mask, tokens, experts, groups, topk_group, topk, renormalize,
                      routed_scaling, logits_dtype, bias_dtype, 0, 0, 0.0, 0, stream);
  }
  MCOP_REQUIRE(routed_scaling != 0.f, MCOP_ERR_ARGUMENT, "moe_gate: routed_scaling must not be 0");
  return gate_entry(logits, bias, topk_weights, topk_ids, group_mask, tokens, experts, groups, topk_group, topk, renormalize,
                    1.0f / routed_scaling, logits_dtype, bias_dtype, 3, num_fused_shared_experts, 0.0, 0, stream);
}

extern "C" int mcop_moe_gate_grouped_sigmoid_shared(const void* logits, const void* bias, float* topk_weights,
                                                    int32_t* topk_ids, int64_t tokens, int experts, int groups,
                                                    int topk_group, int topk, int renormalize, int num_shared_experts,
                                                    double routed_scaling, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(routed_scaling != 0.0, MCOP_ERR_ARGUMENT, "moe_gate: routed_scaling must not be 0");
  return gate_entry(logits, bias, topk_weights, topk_ids, nullptr, tokens, experts, groups, topk_group, topk, renormalize, 1.0f,
                    dtype, dtype, 1, num_shared_experts, 1.0 / routed_scaling, 0, stream);
}

extern "C" int mcop_grouped_topk(const void* scores, const void* bias, float* topk_values, int32_t* topk_ids, int64_t tokens,
                                 int experts, int n_group, int topk_group, int topk, int renormalize, double routed_scaling,
                                 int scoring_func, int scores_dtype, int bias_dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(scoring_func == 0 || scoring_func == 1, MCOP_ERR_ARGUMENT, "grouped_topk: scoring_func must be 0 (none) or 1 (sigmoid)");
  return gate_entry(scores, bias, topk_values, topk_ids, nullptr, tokens, experts, n_group, topk_group, topk, renormalize,
                    (float)routed_scaling, scores_dtype, bias_dtype, 2, 0, 0.0, scoring_func, stream);
}
