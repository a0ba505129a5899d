// The step on the other side of the expert up-projection: SwiGLU + per-row smooth int8 quantisation of rows that
// are grouped by expert (mcoplib.op.moe_swiglu_dynamic_quantize, op/moe_swiglu_dq.cu:63-292).
//
// One CTA per row.  The gate half and the up half of the row (2*H bf16) are read once with 16-byte loads, the
// activated and smoothed values stay in registers across the abs-max reduction, and the int8 row is written once.
#include <math.h>

#include "common.cuh"
#include "tma_pipe.cuh"  // sm_count()

// Sigmoid as the reference kernels compute it, with the fast exponential and the approximate reciprocal
// (op/int8_quant_kernels.cu:1385: val0 * __builtin_mxc_rcpf(1.0f + __builtin_expf(-val0))).  Measured against the IEEE
// expf + division form on 16.8 M elements: codes differ from the CPU restatement on 4.2e-7 of the elements instead of
// 2.4e-7 (tolerance 1e-4), scales to 2.2e-7 either way; the kernels run 20-37 % faster (they are bound by instruction
// issue: exponential, reciprocal and about two dozen other instructions per element).
#define MCOP_SIGMOID(g) __fdividef(1.0f, 1.0f + __expf(-(g)))

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
  const float sig = gate * MCOP_SIGMOID(gate);
  return up * sig * sm;
}

// FULL: the row is exactly THREADS * NVEC vectors of 8 (no bounds test in the unrolled passes)
template <int THREADS, int NVEC, bool FULL>
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
    if (FULL || k < nv) {
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
    if (FULL || k < nv) {
      st_cs_u2(out + k * 8, quant8_rn_unclamped(v[i], mul));
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
  else if (nv == 256) swiglu_quant_vec<128, 2, true><<<grid, 128, 0, s>>>(p);
  else if (nv <= 256) swiglu_quant_vec<128, 2, false><<<grid, 128, 0, s>>>(p);
  else if (nv == 512) swiglu_quant_vec<128, 4, true><<<grid, 128, 0, s>>>(p);
  else if (nv == 896) swiglu_quant_vec<224, 4, true><<<grid, 224, 0, s>>>(p);
  else if (nv == 1024) swiglu_quant_vec<256, 4, true><<<grid, 256, 0, s>>>(p);
  else if (nv <= 1024) swiglu_quant_vec<256, 4, false><<<grid, 256, 0, s>>>(p);
  else if (nv == 2048) swiglu_quant_vec<512, 4, true><<<grid, 512, 0, s>>>(p);
  else if (nv <= 2048) swiglu_quant_vec<512, 4, false><<<grid, 512, 0, s>>>(p);
  else swiglu_quant_vec<1024, 4, false><<<grid, 1024, 0, s>>>(p);
  return check_launch("moe_swiglu_quant_i8");
}

// ---------------------------------------------------------------------------------------------
// SiLU(gate) * up + per-row int8 quantisation without a smooth scale, in the two addressings of
// mcoplib.op.fused_silu_mul_dq_reorder_quant and mcoplib.op.fused_silu_mul_dq_mask_quant
// (op/int8_quant_kernels.cu:881-955, 1355-1417).  One CTA per processed row; the activated values stay in
// registers across the abs-max reduction.
// ---------------------------------------------------------------------------------------------
namespace mcop {
namespace {

struct SiluMulParams {
  const void* x;                 // [rows, 2n]: gate || up
  int64_t rows; int n;
  const void* ids; int ids_i64; int64_t id_lo, id_hi;   // reorder form: row processed iff id in [lo, hi]; null = all
  const void* mask; int mask_i64; int64_t per_group;    // mask form: rows = groups * per_group, row (g, m) iff m < mask[g]
  int8_t* out; int64_t out_row_bytes;                    // codes of row r at out + r * out_row_bytes
  float* scales;                                         // null: the scale is packed into the row at byte n
};

__device__ __forceinline__ int64_t load_index(const void* p, int is_i64, int64_t i) {
  return is_i64 ? reinterpret_cast<const int64_t*>(p)[i] : (int64_t)reinterpret_cast<const int32_t*>(p)[i];
}

__device__ __forceinline__ float silu_mul_value(float gate, float up) {
  return up * (gate * MCOP_SIGMOID(gate));
}

__device__ __forceinline__ void silu_mul_store_scale(const SiluMulParams& p, int64_t row, float amax) {
  const float sc = (float)((double)amax * 0.0078740157);
  if (p.scales) p.scales[row] = sc;
  else *reinterpret_cast<float*>(p.out + row * p.out_row_bytes + p.n) = sc;
}

template <typename T, int THREADS, int NVEC>
__device__ __forceinline__ void silu_mul_row_vec(const SiluMulParams& p, int64_t row, float* red) {
  const int n = p.n, nv = n >> 3;
  const T* g = reinterpret_cast<const T*>(p.x) + row * 2 * (int64_t)n;
  const T* u = g + n;
  float v[NVEC][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int k = threadIdx.x + i * THREADS;
    if (k < nv) {
      float a[8], b[8];
      Vec8<T>::load_nc(g + k * 8, a);
      Vec8<T>::load_nc(u + k * 8, b);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        v[i][q] = silu_mul_value(a[q], b[q]);
        amax = fmaxf(amax, fabsf(v[i][q]));
      }
    }
  }
  amax = block_reduce<true>(amax, red);
  if (threadIdx.x == 0) silu_mul_store_scale(p, row, amax);
  const float mul = amax > 0.f ? 127.0f * (1.0f / amax) : 0.f;
  int8_t* out = p.out + row * p.out_row_bytes;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int k = threadIdx.x + i * THREADS;
    if (k < nv) {
      st_cs_u2(out + k * 8, quant8_rn_unclamped(v[i], mul));
    }
  }
}

template <typename T>
__device__ __forceinline__ void silu_mul_row_any(const SiluMulParams& p, int64_t row, float* red) {
  const int n = p.n;
  const T* g = reinterpret_cast<const T*>(p.x) + row * 2 * (int64_t)n;
  const T* u = g + n;
  float amax = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    amax = fmaxf(amax, fabsf(silu_mul_value(ElemTraits<T>::to_float(g[i]), ElemTraits<T>::to_float(u[i]))));
  amax = block_reduce<true>(amax, red);
  if (threadIdx.x == 0) silu_mul_store_scale(p, row, amax);
  const float mul = amax > 0.f ? 127.0f * (1.0f / amax) : 0.f;
  int8_t* out = p.out + row * p.out_row_bytes;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    out[i] = (int8_t)q_rn_clamp(silu_mul_value(ElemTraits<T>::to_float(g[i]), ElemTraits<T>::to_float(u[i])) * mul, -128, 127);
}

// grid.x walks rows (reorder form) or the rows of group blockIdx.y (mask form)
template <typename T, int THREADS, int NVEC>
__global__ void __launch_bounds__(THREADS) silu_mul_quant_kernel(SiluMulParams p) {
  __shared__ float red[33];
  if (p.mask) {
    const int64_t g = blockIdx.y;
    int64_t cnt = load_index(p.mask, p.mask_i64, g);
    cnt = cnt < 0 ? 0 : (cnt > p.per_group ? p.per_group : cnt);
    for (int64_t m = blockIdx.x; m < cnt; m += gridDim.x) {  // uniform over the CTA
      if constexpr (NVEC > 0) silu_mul_row_vec<T, THREADS, (NVEC > 0 ? NVEC : 1)>(p, g * p.per_group + m, red);
      else silu_mul_row_any<T>(p, g * p.per_group + m, red);
    }
    return;
  }
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    if (p.ids) {
      const int64_t id = load_index(p.ids, p.ids_i64, row);
      if (id < p.id_lo || id > p.id_hi) continue;  // uniform over the CTA
    }
    if constexpr (NVEC > 0) silu_mul_row_vec<T, THREADS, (NVEC > 0 ? NVEC : 1)>(p, row, red);
    else silu_mul_row_any<T>(p, row, red);
  }
}

// One WARP per row, for rows of exactly 32 * NVEC vectors of 8 (n = 1024, 2048): the whole row sits in the warp's
// registers, the abs-max is one warp reduction, and there is no CTA barrier and no bounds test at all; every lane has
// its 2 * NVEC 16-byte loads in flight before the first use.  Same grid conventions as the kernel above, four rows
// per CTA step.
template <typename T, int NVEC>
__global__ void __launch_bounds__(128, 6) silu_mul_quant_warp(SiluMulParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = p.n;
  int64_t base = 0, count = p.rows;
  if (p.mask) {
    const int64_t g = blockIdx.y;
    int64_t cnt = load_index(p.mask, p.mask_i64, g);
    count = cnt < 0 ? 0 : (cnt > p.per_group ? p.per_group : cnt);
    base = g * p.per_group;
  }
  for (int64_t m = (int64_t)blockIdx.x * 4 + warp; m < count; m += (int64_t)gridDim.x * 4) {
    const int64_t row = base + m;
    if (p.ids) {
      const int64_t id = load_index(p.ids, p.ids_i64, row);
      if (id < p.id_lo || id > p.id_hi) continue;  // uniform over the warp
    }
    const T* g = reinterpret_cast<const T*>(p.x) + row * 2 * (int64_t)n;
    const T* u = g + n;
    uint4 ga[NVEC], ub[NVEC];
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      ga[i] = ld_nc_u4(g + (lane + i * 32) * 8);
      ub[i] = ld_nc_u4(u + (lane + i * 32) * 8);
    }
    float v[NVEC][8];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      float a[8], b[8];
      if constexpr (sizeof(T) == 2 && ElemTraits<T>::code == MCOP_BF16) {
        unpack_bf16x8(ga[i], a);
        unpack_bf16x8(ub[i], b);
      } else {
        unpack_f16x8(ga[i], a);
        unpack_f16x8(ub[i], b);
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        v[i][q] = silu_mul_value(a[q], b[q]);
        amax = fmaxf(amax, fabsf(v[i][q]));
      }
    }
    amax = warp_max_nonneg(amax);
    if (lane == 0) silu_mul_store_scale(p, row, amax);
    const float mul = amax > 0.f ? 127.0f * (1.0f / amax) : 0.f;
    int8_t* out = p.out + row * p.out_row_bytes;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) st_cs_u2(out + (lane + i * 32) * 8, quant8_rn_unclamped(v[i], mul));
  }
}

template <typename T>
int launch_silu_mul(const SiluMulParams& p, dim3 grid, bool vec_ok, cudaStream_t s, const char* what) {
  const int nv = p.n >> 3;
  if (vec_ok && (nv == 128 || nv == 256)) {
    // a CTA of this kernel takes four rows per step; it is built for six resident CTAs per SM (80 registers;
    // measured 5.47 TB/s against 5.40 with five CTAs of 96 registers and 5.01 with four)
    const int64_t per_y = p.mask ? p.per_group : p.rows;
    int64_t gx = (per_y + 3) / 4;
    const int64_t cap = p.mask ? 1024 : (int64_t)sm_count() * 6;
    grid.x = (unsigned)(gx < cap ? (gx < 1 ? 1 : gx) : cap);
    if (nv == 128) silu_mul_quant_warp<T, 4><<<grid, 128, 0, s>>>(p);
    else silu_mul_quant_warp<T, 8><<<grid, 128, 0, s>>>(p);
    return check_launch(what);
  }
  if (!vec_ok) silu_mul_quant_kernel<T, 256, 0><<<grid, 256, 0, s>>>(p);
  else if (nv <= 256) silu_mul_quant_kernel<T, 128, 2><<<grid, 128, 0, s>>>(p);
  else if (nv <= 1024) silu_mul_quant_kernel<T, 256, 4><<<grid, 256, 0, s>>>(p);
  else if (nv <= 2048) silu_mul_quant_kernel<T, 512, 4><<<grid, 512, 0, s>>>(p);
  else silu_mul_quant_kernel<T, 1024, 4><<<grid, 1024, 0, s>>>(p);
  return check_launch(what);
}

int dispatch_silu_mul(const SiluMulParams& p, dim3 grid, int dtype, cudaStream_t s, const char* what) {
  const bool vec_ok = p.n % 8 == 0 && aligned16(p.x) && (reinterpret_cast<uintptr_t>(p.out) & 7u) == 0 &&
                      p.out_row_bytes % 8 == 0 && (p.n >> 3) <= 4096;
  switch (dtype) {
    case MCOP_BF16: return launch_silu_mul<__nv_bfloat16>(p, grid, vec_ok, s, what);
    case MCOP_F16: return launch_silu_mul<__half>(p, grid, vec_ok, s, what);
  }
  return set_error(MCOP_ERR_UNSUPPORTED, "%s: activation dtype %d (bf16 or f16 expected)", what, dtype);
}

}  // namespace
}  // namespace mcop

extern "C" int mcop_silu_mul_quant_i8(const void* x, int dtype, const void* row_ids, int ids_are_i64, int64_t id_lo,
                                      int64_t id_hi, int8_t* out, float* scales, int64_t rows, int64_t n,
                                      mcop_stream_t stream) {
  MCOP_REQUIRE(x && out && scales, MCOP_ERR_ARGUMENT, "silu_mul_quant_i8: null pointer");
  MCOP_REQUIRE(rows >= 0 && n > 0 && n <= 0x3fffffff, MCOP_ERR_ARGUMENT, "silu_mul_quant_i8: bad sizes");
  if (rows == 0) return MCOP_OK;
  SiluMulParams p{};
  p.x = x; p.rows = rows; p.n = (int)n;
  p.ids = row_ids; p.ids_i64 = ids_are_i64; p.id_lo = id_lo; p.id_hi = id_hi;
  p.out = out; p.out_row_bytes = n; p.scales = scales;
  // grid-stride over the rows with at most 16 CTAs per SM: fewer, longer-lived CTAs than one per row
  const int64_t cap = (int64_t)sm_count() * 16;
  const int64_t gx = rows < cap ? rows : cap;
  return dispatch_silu_mul(p, dim3((unsigned)gx), dtype, (cudaStream_t)stream, "silu_mul_quant_i8");
}

extern "C" int mcop_silu_mul_quant_i8_masked_pack(const void* x, int dtype, const void* group_counts, int counts_are_i64,
                                                  void* out_packed, int64_t groups, int64_t rows_per_group, int64_t n,
                                                  int64_t out_stride_elems, mcop_stream_t stream) {
  MCOP_REQUIRE(x && group_counts && out_packed, MCOP_ERR_ARGUMENT, "silu_mul_quant_i8_masked_pack: null pointer");
  MCOP_REQUIRE(groups >= 0 && groups <= 65535 && rows_per_group >= 0 && n > 0 && n <= 0x3fffffff && n % 4 == 0, MCOP_ERR_ARGUMENT,
               "silu_mul_quant_i8_masked_pack: bad sizes (at most 65535 groups, n a multiple of 4)");
  MCOP_REQUIRE(out_stride_elems * 2 >= n + 4, MCOP_ERR_ARGUMENT,
               "silu_mul_quant_i8_masked_pack: a row of %lld elements cannot hold %lld codes and the scale",
               (long long)out_stride_elems, (long long)n);
  // the fp32 scale of a row is stored at byte n of its record: records must start on 4-byte boundaries
  MCOP_REQUIRE((reinterpret_cast<uintptr_t>(out_packed) & 3u) == 0 && (out_stride_elems * 2) % 4 == 0, MCOP_ERR_ARGUMENT,
               "silu_mul_quant_i8_masked_pack: out_packed must be 4-byte aligned and out_stride_elems even (the fp32 scale is "
               "stored inside every record)");
  if (groups == 0 || rows_per_group == 0) return MCOP_OK;
  SiluMulParams p{};
  p.x = x; p.rows = groups * rows_per_group; p.n = (int)n;
  p.mask = group_counts; p.mask_i64 = counts_are_i64; p.per_group = rows_per_group;
  p.out = reinterpret_cast<int8_t*>(out_packed); p.out_row_bytes = out_stride_elems * 2; p.scales = nullptr;
  const int64_t gx = rows_per_group < 4096 ? rows_per_group : 4096;
  return dispatch_silu_mul(p, dim3((unsigned)gx, (unsigned)groups), dtype, (cudaStream_t)stream, "silu_mul_quant_i8_masked_pack");
}
