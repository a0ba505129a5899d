// The step on the other side of the expert up-projection: SwiGLU + per-row smooth int8 quantisation of rows that
// are grouped by expert (mcoplib.op.moe_swiglu_dynamic_quantize, op/moe_swiglu_dq.cu:63-292).
//
// One CTA per row.  The gate half and the up half of the row (2*H bf16) are read once with 16-byte loads, the
// activated and smoothed values stay in registers across the abs-max reduction, and the int8 row is written once.
#include <math.h>

#include "common.cuh"

namespace mcop {
namespace {

struct SwigluParams {
  const __nv_bfloat16* x;      // [rows, 2H]: gate || up
  const float* smooth;         // [experts, H]
  const int32_t* starts; const int32_t* counts; int experts;
  int8_t* out; float* scales;  // [rows, H], [rows]
  int hidden;
};

// Expert owning row r (rows of an expert are [starts[e], starts[e] + counts[e])), or -1.
__device__ __forceinline__ int expert_of_row(const SwigluParams& p, int64_t r) {
  int lo = 0, hi = p.experts - 1;
  while (lo < hi) {  // last e with starts[e] <= r
    const int mid = (lo + hi + 1) >> 1;
    if (p.starts[mid] <= r) lo = mid; else hi = mid - 1;
  }
  // (an empty expert shares its start with its successor, and the successor is the later index, so `lo` is the
  // holder whenever the row belongs to anybody)
  return (p.starts[lo] <= r && r < (int64_t)p.starts[lo] + p.counts[lo]) ? lo : -1;
}

__device__ __forceinline__ float swiglu_value(float gate, float up, float sm) {
  const float sig = gate * (1.0f / (1.0f + expf(-gate)));
  return up * sig * sm;
}

template <int THREADS, int NVEC>
__global__ void __launch_bounds__(THREADS) swiglu_quant_vec(SwigluParams p) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const int e = expert_of_row(p, row);
  if (e < 0) return;  // uniform over the CTA
  const int H = p.hidden, nv = H >> 3;
  const __nv_bfloat16* g = p.x + row * 2 * (int64_t)H;
  const __nv_bfloat16* u = g + H;
  const float* sm = p.smooth + (int64_t)e * H;
  float v[NVEC][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int k = threadIdx.x + i * THREADS;
    if (k < nv) {
      float a[8], b[8];
      Vec8<__nv_bfloat16>::load_nc(g + k * 8, a);
      Vec8<__nv_bfloat16>::load_nc(u + k * 8, b);
      const float4 s0 = __ldg(reinterpret_cast<const float4*>(sm + k * 8));
      const float4 s1 = __ldg(reinterpret_cast<const float4*>(sm + k * 8) + 1);
      const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        v[i][q] = swiglu_value(a[q], b[q], s[q]);
        amax = fmaxf(amax, fabsf(v[i][q]));
      }
    }
  }
  amax = block_reduce<true>(amax, red);
  if (threadIdx.x == 0) p.scales[row] = (float)((double)amax * 0.0078740157);
  const float mul = amax > 0.f ? 127.0f * (1.0f / amax) : 0.f;
  int8_t* out = p.out + row * (int64_t)H;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int k = threadIdx.x + i * THREADS;
    if (k < nv) {
      int c[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) c[q] = q_rn_clamp(v[i][q] * mul, -127, 127);
      st_cs_u2(out + k * 8, pack_i8x8(c));
    }
  }
}

__global__ void __launch_bounds__(256) swiglu_quant_any(SwigluParams p) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const int e = expert_of_row(p, row);
  if (e < 0) return;
  const int H = p.hidden;
  const __nv_bfloat16* g = p.x + row * 2 * (int64_t)H;
  const __nv_bfloat16* u = g + H;
  const float* sm = p.smooth + (int64_t)e * H;
  float amax = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    amax = fmaxf(amax, fabsf(swiglu_value(__bfloat162float(g[i]), __bfloat162float(u[i]), sm[i])));
  amax = block_reduce<true>(amax, red);
  if (threadIdx.x == 0) p.scales[row] = (float)((double)amax * 0.0078740157);
  const float mul = amax > 0.f ? 127.0f * (1.0f / amax) : 0.f;
  int8_t* out = p.out + row * (int64_t)H;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[i] = (int8_t)q_rn_clamp(swiglu_value(__bfloat162float(g[i]), __bfloat162float(u[i]), sm[i]) * mul, -127, 127);
}

}  // namespace
}  // namespace mcop

using namespace mcop;

extern "C" int mcop_moe_swiglu_quant_i8(const void* x, const float* smooth, const int32_t* starts, const int32_t* counts,
                                        int8_t* out, float* scales, int64_t rows, int64_t hidden, int experts,
                                        mcop_stream_t stream) {
  MCOP_REQUIRE(x && smooth && starts && counts && out && scales, MCOP_ERR_ARGUMENT, "moe_swiglu_quant_i8: null pointer");
  MCOP_REQUIRE(rows >= 0 && rows <= 0x7fffffffLL && hidden > 0 && hidden <= 0x3fffffff && experts >= 1, MCOP_ERR_ARGUMENT,
               "moe_swiglu_quant_i8: bad sizes");
  if (rows == 0) return MCOP_OK;
  SwigluParams p{reinterpret_cast<const __nv_bfloat16*>(x), smooth, starts, counts, experts, out, scales, (int)hidden};
  const int nv = (int)(hidden >> 3);
  const bool vec_ok = hidden % 8 == 0 && aligned16(x) && aligned16(smooth) && (reinterpret_cast<uintptr_t>(out) & 7u) == 0 && nv <= 4096;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = (unsigned)rows;
  if (!vec_ok) swiglu_quant_any<<<grid, 256, 0, s>>>(p);
  else if (nv <= 256) swiglu_quant_vec<128, 2><<<grid, 128, 0, s>>>(p);
  else if (nv <= 1024) swiglu_quant_vec<256, 4><<<grid, 256, 0, s>>>(p);
  else if (nv <= 2048) swiglu_quant_vec<512, 4><<<grid, 512, 0, s>>>(p);
  else swiglu_quant_vec<1024, 4><<<grid, 1024, 0, s>>>(p);
  return check_launch("moe_swiglu_quant_i8");
}
