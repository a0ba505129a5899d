// Part 3a of the hot path: MoE routers.
//
// Both routers keep a token's expert scores in registers and do every reduction (row max, row sum,
// group top-2, group selection, the k rounds of arg-max) with warp shuffles: no shared memory, no block
// barrier.  Ties always go to the lower index.
#include <math.h>

#include "common.cuh"

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
template <int VPT, int TPR>
__global__ void __launch_bounds__(128) softmax_topk_kernel(float* __restrict__ weights, int32_t* __restrict__ ids,
                                                           const float* __restrict__ logits, int64_t tokens,
                                                           int experts, int k, bool vec_ok) {
  constexpr int ROWS_PER_WARP = 32 / TPR;
  const int lane = threadIdx.x & 31;
  const int g = lane % TPR;
  const int64_t row = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * ROWS_PER_WARP + lane / TPR;
  const bool active = row < tokens;
  const int first = g * VPT;
  float p[VPT];
  if (active && vec_ok) {
    const float4* src = reinterpret_cast<const float4*>(logits + row * experts + first);
#pragma unroll
    for (int i = 0; i < VPT / 4; ++i) {
      const float4 v = __ldg(src + i);
      p[4 * i] = v.x; p[4 * i + 1] = v.y; p[4 * i + 2] = v.z; p[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      p[i] = (active && first + i < experts) ? __ldg(logits + row * experts + first + i) : -INFINITY;
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
      tot += bv;
    }
    if (bi / VPT == g) {
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        if (i == bi % VPT) p[i] = -1.0f;  // probabilities are >= 0
    }
  }
  if (active && g == 0)
    for (int kk = 0; kk < k; ++kk) weights[row * k + kk] = weights[row * k + kk] / tot;
}

template <int VPT, int TPR>
int launch_softmax(float* w, int32_t* ids, const float* logits, int64_t tokens, int experts, int k, cudaStream_t s) {
  constexpr int WARPS = 4;
  const int64_t rows_per_block = WARPS * (32 / TPR);
  const int64_t blocks = (tokens + rows_per_block - 1) / rows_per_block;
  MCOP_REQUIRE(blocks <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "moe_softmax_topk: too many tokens");
  const bool vec_ok = experts == VPT * TPR && aligned16(logits);
  softmax_topk_kernel<VPT, TPR><<<(unsigned)blocks, WARPS * 32, 0, s>>>(w, ids, logits, tokens, experts, k, vec_ok);
  return check_launch("moe_softmax_topk");
}

// ---------------------------------------------------------------------------------------------
// Grouped sigmoid gate.  One warp per token, V = experts / 32 contiguous experts per lane, so a group of
// experts/groups experts is a run of adjacent lanes.
// ---------------------------------------------------------------------------------------------
struct GateParams {
  const void* logits; const void* bias; float* weights; int32_t* ids; int32_t* group_mask;
  int64_t tokens; int experts, groups, topk_group, topk, renormalize; float scaling;
  int t1, ts;  // dtype codes: logits type, and the wider of logits/bias types
};

template <typename T1, typename T2, int V>
__global__ void __launch_bounds__(128) gate_kernel(GateParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= p.tokens) return;  // whole warp leaves together
  const int first = lane * V;
  const T1* x = reinterpret_cast<const T1*>(p.logits) + row * p.experts + first;
  const T2* b = reinterpret_cast<const T2*>(p.bias) + first;
  float score[V], biased[V];
  float xin[V];
  if (sizeof(T1) == 4 && V % 4 == 0) {
#pragma unroll
    for (int i = 0; i < V / 4; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
      xin[4 * i] = v.x; xin[4 * i + 1] = v.y; xin[4 * i + 2] = v.z; xin[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) xin[i] = ElemTraits<T1>::to_float(x[i]);
  }
#pragma unroll
  for (int i = 0; i < V; ++i) {
    score[i] = round_code(1.0f / (1.0f + expf(-xin[i])), p.t1);
    biased[i] = round_code(score[i] + round_code(ElemTraits<T2>::to_float(b[i]), p.ts), p.ts);
  }

  unsigned sel = 0xffffffffu;
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
    const float gscore = round_code(m1 + m2, p.ts);
    const int gid = lane / lpg;
    sel = 0;
    // One warp-wide integer max (redux.sync) on an order-preserving key finds the best remaining group score; the
    // lowest lane holding it belongs to the lowest group index (lanes are ordered by group).
    for (int r = 0; r < p.topk_group; ++r) {
      const unsigned key = ((sel >> gid) & 1u) ? 0u : ordered_key(gscore);
      const unsigned best = __reduce_max_sync(0xffffffffu, key);
      const unsigned who = __ballot_sync(0xffffffffu, key == best);
      const int win = (__ffs(who) - 1) / lpg;
      sel |= 1u << win;
    }
    if (!((sel >> gid) & 1u)) {
#pragma unroll
      for (int i = 0; i < V; ++i) biased[i] = -INFINITY;
    }
    if (p.group_mask && lane == 0) p.group_mask[row] = (int32_t)sel;
  } else if (p.group_mask && lane == 0) {
    p.group_mask[row] = 1;
  }

  float my_w = 0.f;
  int my_id = 0;
  for (int kk = 0; kk < p.topk; ++kk) {
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
#define MCOP_GATE_CASE(V) case V: gate_kernel<T1, T2, V><<<gb, WARPS * 32, 0, s>>>(p); break;
    MCOP_GATE_CASE(1) MCOP_GATE_CASE(2) MCOP_GATE_CASE(4) MCOP_GATE_CASE(6) MCOP_GATE_CASE(8)
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
  cudaStream_t s = (cudaStream_t)stream;
  if (experts <= 8) return launch_softmax<8, 1>(topk_weights, topk_ids, logits, tokens, experts, k, s);
  if (experts <= 16) return launch_softmax<8, 2>(topk_weights, topk_ids, logits, tokens, experts, k, s);
  if (experts <= 32) return launch_softmax<8, 4>(topk_weights, topk_ids, logits, tokens, experts, k, s);
  if (experts <= 64) return launch_softmax<8, 8>(topk_weights, topk_ids, logits, tokens, experts, k, s);
  if (experts <= 128) return launch_softmax<8, 16>(topk_weights, topk_ids, logits, tokens, experts, k, s);
  if (experts <= 256) return launch_softmax<8, 32>(topk_weights, topk_ids, logits, tokens, experts, k, s);
  if (experts <= 512) return launch_softmax<16, 32>(topk_weights, topk_ids, logits, tokens, experts, k, s);
  return launch_softmax<32, 32>(topk_weights, topk_ids, logits, tokens, experts, k, s);
}

extern "C" int mcop_moe_gate_grouped_sigmoid(const void* logits, const void* bias, float* topk_weights,
                                             int32_t* topk_ids, int32_t* group_mask, int64_t tokens, int experts,
                                             int groups, int topk_group, int topk, int renormalize,
                                             float routed_scaling, int logits_dtype, int bias_dtype,
                                             mcop_stream_t stream) {
  MCOP_REQUIRE(logits && bias && topk_weights && topk_ids, MCOP_ERR_ARGUMENT, "moe_gate: null pointer");
  MCOP_REQUIRE(tokens >= 0 && experts > 0 && topk >= 1 && topk <= 32, MCOP_ERR_ARGUMENT, "moe_gate: bad sizes");
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
  GateParams p{logits, bias, topk_weights, topk_ids, group_mask, tokens, experts, groups, topk_group, topk,
               renormalize, routed_scaling, logits_dtype, 0};
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
