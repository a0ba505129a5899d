// Part 1 of the hot path: residual add + RMSNorm (+ per-token int8 quantisation).
//
// One CTA per token row.  The row (and the residual row) is read ONCE with 16-byte loads and kept in
// registers as fp32 across the sum-of-squares reduction, the abs-max reduction and the quantise step, so
// the HBM traffic is the algorithmic minimum: read x and residual, write residual and the int8 codes.
// Rows whose length is not a multiple of 8 elements (or that are not 16-byte aligned) take a scalar
// multi-pass kernel with the same arithmetic.
#include <math.h>

#include <atomic>
#include <initializer_list>
#include <type_traits>

#include "common.cuh"
#include "tma_pipe.cuh"

namespace mcop {
namespace {

enum NormMode {
  kQuant = 0,       // rms_norm_dynamic_per_token_quant: n = T(T(s*r)*w), codes + scale, residual in place
  kFusedAdd = 1,    // fused_add_rms_norm: s = T(x+res), x := n, res := s
  kSmoothQuant = 2, // 9-argument op: divide by r, after_res / after_norm / codes / scale
  kPlain = 3        // rms_norm: out = T(s*d*w)
};

struct NormParams {
  const void* x;
  int64_t x_stride;
  const void* weight;
  const void* smooth;
  const void* residual_in;  // nullable
  void* residual_out;       // where T(x+res) goes (may alias residual_in); nullable
  void* out;                // T output (kFusedAdd: == x; kSmoothQuant: after_norm; kPlain: out)
  int64_t out_stride;
  int8_t* q;
  float* scales;
  const float* scale_ub;
  int hidden;
  float eps;
  int rms_div;
};

// Per-row scalar from the sum of squares.  The squares are accumulated in double, so the mean is the
// correctly rounded fp32 value whatever the summation order; then IEEE fp32 add, sqrt and division
// (the sequence 1/sqrt(var + eps) a host evaluates).
__device__ __forceinline__ float inv_rms(double ss, int hidden, float eps) {
  const float var = (float)(ss / (double)hidden);
  return 1.0f / sqrtf(var + eps);
}

__device__ __forceinline__ double block_sum_f64(double v, double* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (nwarp == 1) return v;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  double r = (lane < nwarp) ? red[lane] : 0.0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}

// FULL: the row is exactly THREADS * NVEC vectors of 8 (hidden 4096 ... 7168 with THREADS = hidden / 32): no bounds
// test in the unrolled passes.
template <typename T, typename WT, int MODE, int THREADS, int NVEC, bool FULL = false>
__global__ void __launch_bounds__(THREADS) norm_rows_vec(NormParams p) {
  __shared__ float red[33];
  __shared__ double red64[33];
  const int64_t row = blockIdx.x;
  const int nv = p.hidden >> 3;
  const T* x = reinterpret_cast<const T*>(p.x) + row * p.x_stride;
  const T* rin = p.residual_in ? reinterpret_cast<const T*>(p.residual_in) + row * (int64_t)p.hidden : nullptr;
  T* rout = p.residual_out ? reinterpret_cast<T*>(p.residual_out) + row * (int64_t)p.hidden : nullptr;
  const WT* w = reinterpret_cast<const WT*>(p.weight);

  float s[NVEC][8];
  double ss = 0.0;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (FULL || v < nv) {
      // x is overwritten by this kernel only in kFusedAdd: use the coherent load there.
      if (MODE == kFusedAdd) Vec8<T>::load(x + v * 8, s[i]); else Vec8<T>::load_nc(x + v * 8, s[i]);
      if (rin) {
        float r[8];
        Vec8<T>::load(rin + v * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) s[i][j] += r[j];
      }
      if (MODE == kFusedAdd) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s[i][j] = round_to<T>(s[i][j]);
      }
      if (rout) Vec8<T>::store(rout + v * 8, s[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fma((double)s[i][j], (double)s[i][j], ss);  // exact product: one instruction, same value
      if (MODE == kSmoothQuant) {
        // the later phases of the reference read the ROUNDED after_res back
#pragma unroll
        for (int j = 0; j < 8; ++j) s[i][j] = round_to<T>(s[i][j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) s[i][j] = 0.f;
    }
  }
  ss = block_sum_f64(ss, red64);
  const float r = inv_rms(ss, p.hidden, p.eps);

  if (MODE == kPlain) {
    const float d = p.rms_div ? 1.0f / r : r;
    T* out = reinterpret_cast<T*>(p.out) + row * p.out_stride;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (FULL || v < nv) {
        float wv[8];
        Vec8<WT>::load_nc(w + v * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) s[i][j] = s[i][j] * d * wv[j];
        Vec8<T>::store(out + v * 8, s[i]);
      }
    }
    return;
  }

  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (FULL || v < nv) {
      float wv[8];
      Vec8<WT>::load_nc(w + v * 8, wv);
      if (MODE == kSmoothQuant) {
        float sm[8];
        Vec8<WT>::load_nc(reinterpret_cast<const WT*>(p.smooth) + v * 8, sm);
        float nw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          nw[j] = s[i][j] / r * wv[j];
          s[i][j] = nw[j] * sm[j];
          amax = fmaxf(amax, fabsf(s[i][j]));
        }
        Vec8<T>::store(reinterpret_cast<T*>(p.out) + row * p.out_stride + v * 8, nw);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s[i][j] = round_to<T>(round_to<T>(s[i][j] * r) * wv[j]);
          amax = fmaxf(amax, fabsf(s[i][j]));
        }
        // kQuant: the normalised row is an optional extra output (sglang's out_bf16)
        if (MODE == kFusedAdd || (MODE == kQuant && p.out)) Vec8<T>::store(reinterpret_cast<T*>(p.out) + row * p.out_stride + v * 8, s[i]);
      }
    }
  }
  if (MODE == kFusedAdd) return;

  amax = block_reduce<true>(amax, red);
  float scale, inv;
  int lo;
  if (MODE == kSmoothQuant) {
    scale = (float)((double)amax / 127.0);
    lo = -127;
  } else {
    if (p.scale_ub) amax = fminf(amax, *p.scale_ub);
    scale = fmaxf(amax / 127.0f, FLT_EPSILON);
    lo = -128;
  }
  inv = 1.0f / scale;
  if (threadIdx.x == 0) p.scales[row] = scale;
  int8_t* q = p.q + row * (int64_t)p.hidden;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (FULL || v < nv) {
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = q_rn_clamp(s[i][j] * inv, lo, 127);
      st_cs_u2(q + v * 8, pack_i8x8(c));
    }
  }
}

// Scalar multi-pass form: any hidden size, any alignment.  Same arithmetic, re-reading the row.
template <typename T, typename WT, int MODE>
__global__ void __launch_bounds__(256) norm_rows_any(NormParams p) {
  __shared__ float red[33];
  __shared__ double red64[33];
  const int64_t row = blockIdx.x;
  const int H = p.hidden;
  const T* x = reinterpret_cast<const T*>(p.x) + row * p.x_stride;
  const T* rin = p.residual_in ? reinterpret_cast<const T*>(p.residual_in) + row * (int64_t)H : nullptr;
  T* rout = p.residual_out ? reinterpret_cast<T*>(p.residual_out) + row * (int64_t)H : nullptr;
  const WT* w = reinterpret_cast<const WT*>(p.weight);
  const WT* sm = reinterpret_cast<const WT*>(p.smooth);
  T* out = p.out ? reinterpret_cast<T*>(p.out) + row * p.out_stride : nullptr;
  // x (kFusedAdd) and the residual row are overwritten in place while later passes need the sum again,
  // so the fp32 sum of the row is parked in shared memory and global memory is read only once.
  extern __shared__ float keep[];  // hidden floats
  double ss = 0.0;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float s = ElemTraits<T>::to_float(x[i]);
    if (rin) s += ElemTraits<T>::to_float(rin[i]);
    if (MODE == kFusedAdd) s = round_to<T>(s);
    if (rout) rout[i] = ElemTraits<T>::from_float(s);
    ss = fma((double)s, (double)s, ss);
    if (MODE == kSmoothQuant) s = round_to<T>(s);
    keep[i] = s;
  }
  ss = block_sum_f64(ss, red64);
  const float r = inv_rms(ss, H, p.eps);
  if (MODE == kPlain) {
    const float d = p.rms_div ? 1.0f / r : r;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      out[i] = ElemTraits<T>::from_float(keep[i] * d * ElemTraits<WT>::to_float(w[i]));
    return;
  }
  float amax = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v;
    if (MODE == kSmoothQuant) {
      const float nw = keep[i] / r * ElemTraits<WT>::to_float(w[i]);
      out[i] = ElemTraits<T>::from_float(nw);
      v = nw * ElemTraits<WT>::to_float(sm[i]);
    } else {
      v = round_to<T>(round_to<T>(keep[i] * r) * ElemTraits<WT>::to_float(w[i]));
      if (MODE == kFusedAdd || (MODE == kQuant && out)) out[i] = ElemTraits<T>::from_float(v);
    }
    keep[i] = v;
    amax = fmaxf(amax, fabsf(v));
  }
  if (MODE == kFusedAdd) return;
  amax = block_reduce<true>(amax, red);
  float scale;
  int lo;
  if (MODE == kSmoothQuant) {
    scale = (float)((double)amax / 127.0);
    lo = -127;
  } else {
    if (p.scale_ub) amax = fminf(amax, *p.scale_ub);
    scale = fmaxf(amax / 127.0f, FLT_EPSILON);
    lo = -128;
  }
  const float inv = 1.0f / scale;
  if (threadIdx.x == 0) p.scales[row] = scale;
  int8_t* q = p.q + row * (int64_t)H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) q[i] = (int8_t)q_rn_clamp(keep[i] * inv, lo, 127);
}


// ---------------------------------------------------------------------------------------------
// Persistent, pipelined form of the bf16 norm + quant kernel (kQuant).
//
// A CTA walks the rows blockIdx.x, blockIdx.x + gridDim.x, ...  The x row and the residual row of the rows
// `stages` ahead are already on their way into shared memory (bulk asynchronous copies completing on an
// mbarrier), so the memory system stays busy while the CTA reduces and quantises the current row.
// Arithmetic is the same as norm_rows_vec<bf16, bf16, kQuant>, written with packed bf16x2 instructions:
// T(s*r) and T(T(s*r)*w) are exactly the roundings cvt.rn.bf16x2 and mul.rn.bf16x2 perform.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t bf16x2_from(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// FULL: the row is exactly THREADS * NVEC vectors of 8, so no lane is ever idle and no pass needs a bounds test.
// LOCKSTEP selects how the warps of the CTA are kept together (both forms compute the same values):
//   false - two CTA barriers per row: the per-warp partial results of the two reductions go to shared-memory slots
//           that alternate between consecutive rows, so neither reduction needs a trailing barrier;
//   true  - a barrier before the stage is read and the classic two-barrier block reductions (five per row).
// Measured on B200: with 7 warps (hidden 7168) the loose form is 6 % faster (6.36 vs 5.97 TB/s); with 8 warps
// (hidden 8192) the lock-step form is 14 % faster (6.26 vs 5.50 TB/s), so the launcher picks per CTA size.
// PMODE 0: norm + per-token int8 quant (a2 contract: the variance is taken from the unrounded fp32 sum).
// PMODE 1: fused_add_rms_norm (a1 contract: r = bf16(x + res) is rounded BEFORE the variance; the normalised row
//          bf16(bf16(r * rsqrt) * w) goes to p.out, which is x itself; nothing is quantised and the row needs one
//          barrier less).
// PMODE 2: rms_norm (a4 contract: fp32 products (s * d) * w with d = rsqrt or, with rms_div, its reciprocal; one rounding;
//          residual and after_res optional).
// PMODE 3: the 9-argument norm + smooth quant (a3 contract: after_res = bf16(x + res) always written; the variance from
//          the unrounded sum; nw = (after_res / rsqrt) * w with after_res read back ROUNDED, after_norm = bf16(nw);
//          y = nw * smooth; scale = absmax(y) / 127; codes clamped to +-127).
template <int THREADS, int NVEC, bool FULL, bool LOCKSTEP, bool NORM_OUT, int PMODE = 0>
__global__ void __launch_bounds__(THREADS, (THREADS <= 256 ? 2 : 1)) norm_quant_bf16_pipe(NormParams p, int64_t tokens, int stages, int* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float red[2][32];
  __shared__ __align__(16) double red64[2][32];
  constexpr int NWARP = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // `stages` (<= 8) barriers in the first 128 bytes
  unsigned char* buf = smem + 128;
  const int H = p.hidden, nv = H >> 3;
  const uint32_t row_bytes = (uint32_t)H * 2u;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x);
  const __nv_bfloat16* rin = reinterpret_cast<const __nv_bfloat16*>(p.residual_in);
  __nv_bfloat16* rout = reinterpret_cast<__nv_bfloat16*>(p.residual_out);
  const bool has_res = rin != nullptr;
  const uint32_t stage_bytes = has_res ? 2u * row_bytes : row_bytes;
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t n = first < tokens ? (tokens - first + step - 1) / step : 0;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();
  pdl_wait();  // nothing of global memory is touched before the kernels ahead in the stream have completed
  auto issue = [&](int s, int64_t row) {
    unsigned char* dst = buf + (size_t)s * stage_bytes;
    mbar_expect_tx(&full[s], stage_bytes);
    bulk_g2s(dst, x + row * p.x_stride, row_bytes, &full[s]);
    if (has_res) bulk_g2s(dst + row_bytes, rin + row * (int64_t)H, row_bytes, &full[s]);
  };
  if (threadIdx.x == 0)
    for (int s = 0; s < stages && s < n; ++s) issue(s, first + s * step);

  // the norm weight stays in registers, packed as bf16 pairs, for every row this CTA handles
  uint4 w2[NVEC];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    w2[i] = (FULL || v < nv) ? ld_nc_u4(reinterpret_cast<const __nv_bfloat16*>(p.weight) + v * 8) : make_uint4(0, 0, 0, 0);
  }

  uint4 sm2[PMODE == 3 ? NVEC : 1];  // PMODE 3: the smooth scale too
  if constexpr (PMODE == 3) {
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * THREADS;
      sm2[i] = (FULL || v < nv) ? ld_nc_u4(reinterpret_cast<const __nv_bfloat16*>(p.smooth) + v * 8) : make_uint4(0, 0, 0, 0);
    }
  }

  bool wnan = false;  // PMODE 3: a NaN among this thread's weights or smooth scales (checked once, not per row)
  if constexpr (PMODE == 3) {
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
      float a[8], b[8];
      unpack_bf16x8(w2[k], a);
      unpack_bf16x8(sm2[k], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) wnan |= (a[j] != a[j]) | (b[j] != b[j]);
    }
  }

  int64_t i = 0;
  RingPos pos;
  uint32_t flip = 0;
  for (; i < n; ++i, pos.advance(stages), flip ^= 1u) {
    const int s = pos.s;
    const bool ok = mbar_wait_bounded(&full[s], pos.phase, err, 1);
    if constexpr (LOCKSTEP) {
      if (!__syncthreads_and(ok)) break;  // uniform decision: nobody is left behind at a barrier
    }
    const int64_t row = first + i * step;
    const unsigned char* xs = buf + (size_t)s * stage_bytes;
    float sv[NVEC][8];
    double ss = 0.0;
    if (ok)  // when the wait ran out the stage is not read; the next barrier then ends the loop for everybody
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
      const int v = threadIdx.x + k * THREADS;
      if (FULL || v < nv) {
        uint4 packed = lds_u4(xs + v * 16);
        unpack_bf16x8(packed, sv[k]);
        if (has_res) {
          float r[8];
          unpack_bf16x8(lds_u4(xs + row_bytes + v * 16), r);
#pragma unroll
          for (int j = 0; j < 8; ++j) sv[k][j] += r[j];
          packed = pack_bf16x8(sv[k]);
          if (PMODE != 2 || rout) st_u4(rout + row * (int64_t)H + v * 8, packed);  // (rms_norm's after_res is optional)
          if constexpr (PMODE == 1) unpack_bf16x8(packed, sv[k]);  // the rounded sum is what gets normalised
        } else if constexpr (PMODE == 3) {
          st_u4(rout + row * (int64_t)H + v * 8, packed);  // after_res is written even without a residual (= x)
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fma((double)sv[k][j], (double)sv[k][j], ss);  // the product is exact in double
        if constexpr (PMODE == 3) unpack_bf16x8(packed, sv[k]);  // the later phases read the ROUNDED after_res back
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) sv[k][j] = 0.f;
      }
    }
    if constexpr (LOCKSTEP) {
      ss = block_sum_f64(ss, &red64[0][0]);  // its barrier also tells that every thread has left the stage buffer
    } else {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) red64[flip][warp] = ss;
      // first barrier of the row: agrees on success, publishes the warps' partial sums and tells that every thread
      // has left the stage buffer
      if (!__syncthreads_and(ok)) break;
    }
    if (threadIdx.x == 0 && i + stages < n) {
      proxy_fence_before_reuse();
      issue(s, first + (i + stages) * step);
    }
    if constexpr (!LOCKSTEP) {
      ss = lane < NWARP ? red64[flip][lane] : 0.0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    const float r = inv_rms(ss, H, p.eps);
    if constexpr (PMODE == 2) {
      const float d = p.rms_div ? 1.0f / r : r;
#pragma unroll
      for (int k = 0; k < NVEC; ++k) {
        const int v = threadIdx.x + k * THREADS;
        if (FULL || v < nv) {
          float wf[8], o[8];
          unpack_bf16x8(w2[k], wf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = __fmul_rn(__fmul_rn(sv[k][j], d), wf[j]);
          st_u4(reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.out_stride + v * 8, pack_bf16x8(o));
        }
      }
      continue;
    }
    uint32_t n2[NVEC][4];
    __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.f, 0.f);
    float amax3 = 0.f;
    const bool r_ok3 = r >= 9.31322574615478515625e-10f && r <= 1073741824.0f;  // (PMODE 3) 2^-30 .. 2^30, not a NaN
    if constexpr (PMODE == 3) {
      // literal convention of the 9-argument operator: divide by rsqrt; after_norm = T(nw), y = nw * smooth stays fp32.
      // The quotients s / r of a row share the divisor: with inv = rn(1 / r), q0 = rn(s * inv) corrected twice by
      // q + rn(s - q * r) * inv is the correctly rounded quotient (the first step makes q faithful, the second rounds it
      // correctly: Markstein), five packed operations per pair instead of two division sequences.  Every intermediate must
      // stay in the normal range: rows whose r is outside 2^-30 .. 2^30 (or a NaN) and vectors with an element below 2^-60
      // (a zero counts: merely slower) take the division itself.
      const bool r_ok = r_ok3;
      const float inv_r = __frcp_rn(r);
      const float2 inv2 = make_float2(inv_r, inv_r), nr2 = make_float2(-r, -r);
#pragma unroll
      for (int k = 0; k < NVEC; ++k) {
        const int v = threadIdx.x + k * THREADS;
        if (FULL || v < nv) {
          float wf[8], sf[8], nw[8];
          unpack_bf16x8(w2[k], wf);
          unpack_bf16x8(sm2[k], sf);
          float amin = min3_abs(sv[k][0], sv[k][1], 1.0f);
#pragma unroll
          for (int j = 2; j < 8; j += 2) amin = min3_abs(sv[k][j], sv[k][j + 1], amin);
          if (r_ok && amin >= 8.67361737988403547206e-19f) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const float2 a = make_float2(sv[k][j], sv[k][j + 1]);
              const float2 q0 = mul2_rn(a, inv2);
              const float2 q1 = __ffma2_rn(__ffma2_rn(q0, nr2, a), inv2, q0);
              const float2 q2 = __ffma2_rn(__ffma2_rn(q1, nr2, a), inv2, q1);
              const float2 n2v = mul2_rn(q2, make_float2(wf[j], wf[j + 1]));
              const float2 y2 = mul2_rn(n2v, make_float2(sf[j], sf[j + 1]));
              nw[j] = n2v.x; nw[j + 1] = n2v.y;
              sv[k][j] = y2.x; sv[k][j + 1] = y2.y;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              nw[j] = __fmul_rn(__fdiv_rn(sv[k][j], r), wf[j]);
              sv[k][j] = __fmul_rn(nw[j], sf[j]);
            }
          }
#pragma unroll
          for (int j = 0; j < 8; j += 2) amax3 = max3_abs(sv[k][j], sv[k][j + 1], amax3);
          st_u4(reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.out_stride + v * 8, pack_bf16x8(nw));
        }
      }
    } else
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
      const uint32_t wv[4] = {w2[k].x, w2[k].y, w2[k].z, w2[k].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t t = bf16x2_from(sv[k][2 * j] * r, sv[k][2 * j + 1] * r);
        const __nv_bfloat162 nn = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&t), *reinterpret_cast<const __nv_bfloat162*>(&wv[j]));
        n2[k][j] = *reinterpret_cast<const uint32_t*>(&nn);
        amax2 = __hmax2(amax2, __habs2(nn));
      }
    }
    if constexpr (PMODE == 1) {
#pragma unroll
      for (int k = 0; k < NVEC; ++k) {
        const int v = threadIdx.x + k * THREADS;
        if (FULL || v < nv)
          st_u4(reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.out_stride + v * 8, make_uint4(n2[k][0], n2[k][1], n2[k][2], n2[k][3]));
      }
      continue;
    }
    float amax = PMODE == 3 ? amax3 : fmaxf(__low2float(amax2), __high2float(amax2));  // never negative, never NaN
    if constexpr (LOCKSTEP) {
      amax = block_reduce<true>(amax, &red[0][0]);
    } else {
      amax = warp_max_nonneg(amax);
      if (lane == 0) red[flip][warp] = amax;
      __syncthreads();  // second barrier of the row
      amax = warp_max_nonneg(lane < NWARP ? red[flip][lane] : 0.f);
    }
    if constexpr (PMODE == 3) {
      const float scale3 = (float)((double)amax / 127.0);
      const float inv3 = 1.0f / scale3;
      if (threadIdx.x == 0) p.scales[row] = scale3;
      int8_t* q3 = p.q + row * (int64_t)H;
      // |y * inv3| <= 127 * (1 + 2^-22) for every finite row with a normal scale: no clamp, and the fp32 adder rounds
      // (eight conversions per vector on the quarter-rate conversion unit otherwise).  Rows with a NaN or an infinity
      // (r is then outside its range), a zero, tiny or huge scale, or a NaN in this thread's weights keep the conversion.
      if (r_ok3 && !wnan && scale3 >= 7.888609e-31f && scale3 <= 1.2676506e30f) {
#pragma unroll
        for (int k = 0; k < NVEC; ++k) {
          const int v = threadIdx.x + k * THREADS;
          if (FULL || v < nv) st_cs_u2(q3 + v * 8, quant8_rn_unclamped(sv[k], inv3));
        }
      } else {
#pragma unroll
        for (int k = 0; k < NVEC; ++k) {
          const int v = threadIdx.x + k * THREADS;
          if (FULL || v < nv) {
            int c[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) c[j] = q_rn_clamp(sv[k][j] * inv3, -127, 127);
            st_cs_u2(q3 + v * 8, pack_i8x8(c));
          }
        }
      }
      continue;
    }
    const bool clamp = p.scale_ub != nullptr;  // only an upper bound on the scale can push codes out of range
    if (clamp) amax = fminf(amax, *p.scale_ub);
    const float scale = fmaxf(amax / 127.0f, FLT_EPSILON);
    const float inv = 1.0f / scale;
    if (threadIdx.x == 0) p.scales[row] = scale;
    int8_t* q = p.q + row * (int64_t)H;
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
      const int v = threadIdx.x + k * THREADS;
      if (FULL || v < nv) {
        uint32_t c[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a = __fmul_rn(__uint_as_float(n2[k][j] << 16), inv);
          float b = __fmul_rn(__uint_as_float(n2[k][j] & 0xffff0000u), inv);
          if (clamp) {
            a = fminf(fmaxf(a, -128.f), 127.f);
            b = fminf(fmaxf(b, -128.f), 127.f);
          }
          c[2 * j] = rn_low_byte(a);      // without a bound |n * inv| <= 127 * (1 + 2^-22): always in range
          c[2 * j + 1] = rn_low_byte(b);
        }
        st_cs_u2(q + v * 8, make_uint2(pack4_low_bytes(c[0], c[1], c[2], c[3]), pack4_low_bytes(c[4], c[5], c[6], c[7])));
        // optional extra output, the normalised bf16 row: a compile-time variant because a run-time test of p.out here
        // costs the plain form 3-4 % (6.13 against 6.38 TB/s at hidden 7168, measured on one box)
        if constexpr (NORM_OUT)
          st_u4(reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.out_stride + v * 8, make_uint4(n2[k][0], n2[k][1], n2[k][2], n2[k][3]));
      }
    }
  }
  if (i < n && threadIdx.x == 0) {
    // a wait ran out: drain (bounded) what is still in flight so that no copy lands after the CTA has exited
    for (int64_t k = i; k < n && k < i + stages; ++k, pos.advance(stages))
      (void)mbar_wait_bounded(&full[pos.s], pos.phase, err, 2);
  }
}


// Returns MCOP_OK / an error, or 1 when the shape does not fit the pipelined kernel.
template <int PMODE>
inline int launch_norm_pipe(const NormParams& p, int64_t tokens, cudaStream_t stream) {
  const int nv = p.hidden >> 3;
  const size_t row_bytes = (size_t)p.hidden * 2;
  const size_t stage_bytes = p.residual_in ? 2 * row_bytes : row_bytes;
  int stages = (int)((110 * 1024) / stage_bytes);
  stages = stages < 2 ? 2 : (stages > 4 ? 4 : stages);
  const size_t smem = 128 + (size_t)stages * stage_bytes;
  if (smem > 220 * 1024) return 1;
  // 4 to 7 warps when they tile the row exactly (hidden 4096 ... 7168 = 4 x 128 ... 224 vectors of 8), else 8 or 16
  const bool tiles = nv == 512 || nv == 640 || nv == 768 || nv == 896;
  const int threads = tiles ? nv / 4 : ((nv <= 896 && nv % 224 == 0) ? 224 : (nv <= 1024 ? 256 : 512));
  const bool full = nv == threads * 4;
  int per_sm = (int)((227 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : per_sm;
  if (per_sm > 2048 / threads) per_sm = 2048 / threads;
  if (per_sm > 4) per_sm = 4;
  int64_t grid = (int64_t)sm_count() * per_sm;
  if (grid > tokens) grid = tokens;
  int* err = pipe_error_ptr();
  const bool no = PMODE == 0 && p.out != nullptr;  // also write the normalised row
  auto launch = [&](auto kernel, int) -> int {
    const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), 220 * 1024);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "norm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    (void)launch_pdl(kernel, dim3((unsigned)grid), dim3(threads), smem, stream, p, tokens, stages, err);
    return check_launch("norm (pipelined)");
  };
#define MCOP_NORM_TILED(T, SLOT)                                                                        \
  if (threads == T && full && T != 224)                                                                 \
    return no ? launch(norm_quant_bf16_pipe<T, 4, true, false, true, PMODE>, SLOT) : launch(norm_quant_bf16_pipe<T, 4, true, false, false, PMODE>, SLOT + 1);
  MCOP_NORM_TILED(128, 8)
  MCOP_NORM_TILED(160, 10)
  MCOP_NORM_TILED(192, 12)
#undef MCOP_NORM_TILED
  if (threads == 224) {
    if (full) return no ? launch(norm_quant_bf16_pipe<224, 4, true, false, true, PMODE>, 0) : launch(norm_quant_bf16_pipe<224, 4, true, false, false, PMODE>, 1);
    return no ? launch(norm_quant_bf16_pipe<224, 4, false, false, true, PMODE>, 2) : launch(norm_quant_bf16_pipe<224, 4, false, false, false, PMODE>, 3);
  }
  if (threads == 256)
    return no ? launch(norm_quant_bf16_pipe<256, 4, false, true, true, PMODE>, 4) : launch(norm_quant_bf16_pipe<256, 4, false, true, false, PMODE>, 5);
  return no ? launch(norm_quant_bf16_pipe<512, 4, false, true, true, PMODE>, 6) : launch(norm_quant_bf16_pipe<512, 4, false, true, false, PMODE>, 7);
}

template <typename T, typename WT, int MODE>
int launch_norm(const NormParams& p, int64_t tokens, bool vec_ok, cudaStream_t stream) {
  if (tokens == 0) return MCOP_OK;
  MCOP_REQUIRE(tokens <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "norm: %lld tokens exceed the grid limit", (long long)tokens);
  const int nv = p.hidden >> 3;
  const dim3 grid((unsigned)tokens);
  if constexpr (MODE == kQuant && std::is_same<T, __nv_bfloat16>::value) {
    if (vec_ok && nv <= 2048) {
      const int rc = launch_norm_pipe<0>(p, tokens, stream);
      if (rc != 1) return rc;  // 1 = not applicable, fall through to the row-per-CTA kernel
    }
  }
  if constexpr (MODE == kSmoothQuant && std::is_same<T, __nv_bfloat16>::value && std::is_same<WT, __nv_bfloat16>::value) {
    if (vec_ok && nv >= 256 && nv <= 2048 && tokens >= 1024) {
      const int rc = launch_norm_pipe<3>(p, tokens, stream);
      if (rc != 1) return rc;
    }
  }
  if constexpr (MODE == kPlain && std::is_same<T, __nv_bfloat16>::value && std::is_same<WT, __nv_bfloat16>::value) {
    if (vec_ok && nv >= 256 && nv <= 2048 && tokens >= 1024) {
      const int rc = launch_norm_pipe<2>(p, tokens, stream);
      if (rc != 1) return rc;
    }
  }
  if constexpr (MODE == kFusedAdd && std::is_same<T, __nv_bfloat16>::value && std::is_same<WT, __nv_bfloat16>::value) {
    // a1 on bf16 rows streams through the same ring as a2 once there are a few waves of rows
    if (vec_ok && nv <= 2048 && p.residual_in && tokens >= 1024) {
      const int rc = launch_norm_pipe<1>(p, tokens, stream);
      if (rc != 1) return rc;
    }
  }
  if (vec_ok && nv <= 4096) {
    if (nv <= 256) norm_rows_vec<T, WT, MODE, 128, 2><<<grid, 128, 0, stream>>>(p);
    else if (nv == 512) norm_rows_vec<T, WT, MODE, 128, 4, true><<<grid, 128, 0, stream>>>(p);
    else if (nv == 640) norm_rows_vec<T, WT, MODE, 160, 4, true><<<grid, 160, 0, stream>>>(p);
    else if (nv == 768) norm_rows_vec<T, WT, MODE, 192, 4, true><<<grid, 192, 0, stream>>>(p);
    else if (nv == 896) norm_rows_vec<T, WT, MODE, 224, 4, true><<<grid, 224, 0, stream>>>(p);
    else if (nv <= 1024) norm_rows_vec<T, WT, MODE, 256, 4><<<grid, 256, 0, stream>>>(p);
    else if (nv <= 2048) norm_rows_vec<T, WT, MODE, 512, 4><<<grid, 512, 0, stream>>>(p);
    else norm_rows_vec<T, WT, MODE, 1024, 4><<<grid, 1024, 0, stream>>>(p);
  } else {
    const size_t smem = (size_t)p.hidden * sizeof(float);
    MCOP_REQUIRE(smem <= 200 * 1024, MCOP_ERR_UNSUPPORTED, "norm: hidden %d too large for the unaligned path", p.hidden);
    if (smem > 48 * 1024) {
      const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&norm_rows_any<T, WT, MODE>), smem);
      MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "norm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    norm_rows_any<T, WT, MODE><<<grid, 256, smem, stream>>>(p);
  }
  return check_launch("norm");
}

// Weight type choices: same as the activation type, or fp32.
template <typename T, int MODE>
int dispatch_wt(const NormParams& p, int64_t tokens, bool vec_ok, int dtype, int wdtype, cudaStream_t stream) {
  if (wdtype == dtype) return launch_norm<T, T, MODE>(p, tokens, vec_ok, stream);
  if (wdtype == MCOP_F32) return launch_norm<T, float, MODE>(p, tokens, vec_ok, stream);
  return set_error(MCOP_ERR_UNSUPPORTED, "norm: weight dtype %d with activation dtype %d", wdtype, dtype);
}

template <int MODE>
int dispatch_norm(const NormParams& p, int64_t tokens, bool vec_ok, int dtype, int wdtype, cudaStream_t stream) {
  constexpr bool same_only = (MODE == kQuant || MODE == kFusedAdd);
  if (same_only) {
    MCOP_REQUIRE(wdtype == dtype, MCOP_ERR_UNSUPPORTED, "norm: weight dtype must equal the activation dtype");
    switch (dtype) {
      case MCOP_BF16: return launch_norm<__nv_bfloat16, __nv_bfloat16, MODE>(p, tokens, vec_ok, stream);
      case MCOP_F16: return launch_norm<__half, __half, MODE>(p, tokens, vec_ok, stream);
      case MCOP_F32: return launch_norm<float, float, MODE>(p, tokens, vec_ok, stream);
    }
  } else {
    switch (dtype) {
      case MCOP_BF16: return dispatch_wt<__nv_bfloat16, MODE>(p, tokens, vec_ok, dtype, wdtype, stream);
      case MCOP_F16: return dispatch_wt<__half, MODE>(p, tokens, vec_ok, dtype, wdtype, stream);
      case MCOP_F32: return dispatch_wt<float, MODE>(p, tokens, vec_ok, dtype, wdtype, stream);
    }
  }
  return set_error(MCOP_ERR_UNSUPPORTED, "norm: unknown dtype code %d", dtype);
}

inline int elem_size(int dtype) { return dtype == MCOP_F32 ? 4 : 2; }

bool rows_vectorisable(int64_t hidden, int dtype, int wdtype, const void* x, int64_t x_stride,
                       std::initializer_list<const void*> contiguous_t, std::initializer_list<const void*> w_ptrs,
                       const void* q) {
  if (hidden % 8) return false;
  if (!aligned16(x) || (x_stride * elem_size(dtype)) % 16) return false;
  for (const void* p : contiguous_t) if (p && !aligned16(p)) return false;
  for (const void* p : w_ptrs) if (p && !aligned16(p)) return false;
  if (q && (reinterpret_cast<uintptr_t>(q) & 7u)) return false;
  (void)wdtype;
  return true;
}

// ---------------------------------------------------------------------------------------------
// head_rms_norm: one warp per (token, head); divide-by-rsqrt convention.
// ---------------------------------------------------------------------------------------------
template <typename T, typename WT>
__global__ void head_rmsnorm_kernel(T* out, const T* x, const WT* w, int64_t tokens, int heads, int head_dim,
                                    float eps, int head_offset, int head_norm) {
  const int warps = blockDim.x >> 5;
  const int64_t item = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5);
  if (item >= tokens * head_norm) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = item / head_norm;
  const int h = head_offset + (int)(item % head_norm);
  const T* src = x + (t * heads + h) * (int64_t)head_dim;
  T* dst = out + (t * heads + h) * (int64_t)head_dim;
  const WT* wh = w + (int64_t)h * head_dim;
  double ss = 0.0;
  for (int i = lane; i < head_dim; i += 32) {
    const float v = ElemTraits<T>::to_float(src[i]);
    ss = fma((double)v, (double)v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = inv_rms(ss, head_dim, eps);
  for (int i = lane; i < head_dim; i += 32)
    dst[i] = ElemTraits<T>::from_float(ElemTraits<T>::to_float(src[i]) / r * ElemTraits<WT>::to_float(wh[i]));
}

// The same with 16-byte accesses, for heads of 8 * G elements (G = 8, 16 or 32 lanes per head: head_dim 64, 128, 256).
// A warp takes 32 / G heads per turn and walks the heads with a grid stride; the vector of the next turn is loaded before
// the current one is reduced, and token / head of a turn follow from the previous turn by an add and a carry (the stride's
// quotient and remainder by head_norm come from the host) instead of a division per head.
//
// The kernel is bound by instruction issue, not by memory, so the eight quotients x / r of a lane (one divisor) are not
// eight IEEE division sequences: with inv = rn(1 / r), q0 = rn(x * inv) is within two ulps of x / r; one step
// q1 = rn(q0 + rn(x - q0 * r) * inv) (the residual is exact in a fused multiply-add) makes it a faithful rounding, and a
// second step the correctly rounded quotient (Markstein's theorem: a faithful quotient corrected with the correctly
// rounded reciprocal rounds correctly), five packed operations per pair of elements.  That argument needs every
// intermediate in the normal range, so the lane's vector goes through the division itself when r is outside
// [2^-30, 2^30] (also a NaN r) or an element is nonzero and below 2^-60 (|x| <= sqrt(D) / r bounds the elements from
// above).  The mean of squares is ss * (1 / D): D is a power of two, the product equals the quotient.
__device__ __forceinline__ uint4 ld_nc_keep_u4(const void* p) {  // read-only path, kept in L1 (the weight table)
  uint4 r;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
template <typename WT> __device__ __forceinline__ void load_weight8(const WT* p, float (&v)[8]) {
  if constexpr (sizeof(WT) == 4) {
    const uint4 a = ld_nc_keep_u4(p), b = ld_nc_keep_u4(p + 4);
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
  } else if constexpr (ElemTraits<WT>::code == MCOP_BF16) {
    unpack_bf16x8(ld_nc_keep_u4(p), v);
  } else {
    unpack_f16x8(ld_nc_keep_u4(p), v);
  }
}

template <typename T, typename WT, int G>
__global__ void __launch_bounds__(256) head_rmsnorm_vec(T* out, const T* x, const WT* w, int64_t total, int heads, float eps,
                                                        int head_offset, int head_norm, int64_t stride_tokens, int stride_heads) {
  constexpr int HPW = 32 / G;  // heads per warp and turn
  constexpr int D = 8 * G;
  const int lane = threadIdx.x & 31, gl = lane % G;
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  int64_t item = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * HPW + lane / G;
  const int64_t step = nwarps * HPW;  // = stride_tokens * head_norm + stride_heads
  // token and head of the first turn: the one division of the thread
  int64_t t = item / head_norm;
  int h = (int)(item - t * head_norm);
  float cur[8], nxt[8];
  auto load = [&](float (&v)[8], int64_t tt, int hh) { Vec8<T>::load_nc(x + (tt * heads + head_offset + hh) * (int64_t)D + gl * 8, v); };
  if (item < total) load(cur, t, h);
  else
#pragma unroll
    for (int j = 0; j < 8; ++j) cur[j] = 0.f;
  for (; __any_sync(0xffffffffu, item < total); item += step) {
    const bool live = item < total;
    // the turn after this one
    int64_t tn = t + stride_tokens;
    int hn = h + stride_heads;
    if (hn >= head_norm) { hn -= head_norm; ++tn; }
    if (item + step < total) load(nxt, tn, hn);
    else
#pragma unroll
      for (int j = 0; j < 8; ++j) nxt[j] = 0.f;

    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fma((double)cur[j], (double)cur[j], ss);
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (live) {
      const float var = (float)(ss * (1.0 / D));
      const float r = 1.0f / sqrtf(var + eps);
      float wv[8], o8[8];
      load_weight8(w + (int64_t)(head_offset + h) * D + gl * 8, wv);
      bool exact = !(r >= 9.31322574615478515625e-10f && r <= 1073741824.0f);  // outside 2^-30 .. 2^30, or a NaN
#pragma unroll
      for (int j = 0; j < 8; ++j) exact |= (fabsf(cur[j]) < 8.67361737988403547206e-19f) & (cur[j] != 0.f);  // below 2^-60
      if (!exact) {
        const float inv = __frcp_rn(r);
        const float2 inv2 = make_float2(inv, inv), nr2 = make_float2(-r, -r);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float2 a = make_float2(cur[j], cur[j + 1]);
          const float2 q0 = mul2_rn(a, inv2);
          const float2 q1 = __ffma2_rn(__ffma2_rn(q0, nr2, a), inv2, q0);
          const float2 q2 = __ffma2_rn(__ffma2_rn(q1, nr2, a), inv2, q1);
          const float2 nw = mul2_rn(q2, make_float2(wv[j], wv[j + 1]));
          o8[j] = nw.x;
          o8[j + 1] = nw.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o8[j] = __fmul_rn(__fdiv_rn(cur[j], r), wv[j]);   // the divide-by-rsqrt convention
      }
      Vec8<T>::store(out + (t * heads + head_offset + h) * (int64_t)D + gl * 8, o8);
    }
    t = tn;
    h = hn;
#pragma unroll
    for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
  }
}

// Persistent, pipelined form for many tokens.  The heads to normalise of one token are one contiguous run of
// head_norm * D elements; a CTA walks the tokens blockIdx.x, blockIdx.x + gridDim.x, ... with the runs of the tokens
// `stages` ahead on their way into shared memory (bulk asynchronous copies completing on an mbarrier): the loads of the
// kernel above are one 16-byte vector per lane and turn, too few bytes in flight to cover the memory latency (3.5 TB/s).
//
// A head of D = 8 * G * V elements is held by G lanes with V vectors of 8 each (vector c of lane g is vector c * G + g of
// the head), so a warp takes 32 / G heads per round and a lane has R rounds per token.  Which heads a lane works on does
// not depend on the token: their weights stay in registers (R * V <= 4 vectors).  What costs here is instructions, not
// bytes (sqrt, two reciprocals, the 64-bit shuffles and the address arithmetic are per head and lane): with V = 1 a
// lane-head of 8 elements costs 165 warp instructions, 20 per element, and the kernel runs at 4 TB/s with half of the
// issue slots used; V = 4 spreads the per-head part over 32 elements (5.4 TB/s at 56 heads of 128; 118 registers, two
// CTAs per SM - capped at 80 registers for three CTAs it spills and measured 7 % slower).  Same arithmetic as above, the tiny-element test
// folded into one three-input minimum per pair (a zero element sends its lane through the division too: merely slower).
template <typename T, typename WT, int G, int V>
__global__ void __launch_bounds__(256, (V == 4 ? 2 : 3)) head_rmsnorm_pipe(T* out, const T* x, const WT* w, int64_t tokens, int heads, float eps,
                                                            int head_offset, int head_norm, int stages, int* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int HPW = 32 / G, D = 8 * G * V, R = 4 / V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5, gl = lane % G;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // `stages` (<= 8) barriers in the first 128 bytes
  unsigned char* buf = smem + 128;
  const uint32_t row_bytes = (uint32_t)head_norm * D * (uint32_t)sizeof(T);
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t n = first < tokens ? (tokens - first + step - 1) / step : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();
  auto issue = [&](int s, int64_t t) {
    mbar_expect_tx(&full[s], row_bytes);
    bulk_g2s(buf + (size_t)s * row_bytes, x + (t * heads + head_offset) * (int64_t)D, row_bytes, &full[s]);
  };
  if (threadIdx.x == 0)
    for (int s = 0; s < stages && s < n; ++s) issue(s, first + s * step);

  // round k of this lane works on head (k * nwarp + warp) * HPW + lane / G of the run
  float wv[R][V][8];
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int h = (k * nwarp + warp) * HPW + lane / G;
#pragma unroll
    for (int c = 0; c < V; ++c) {
      if (h < head_norm) load_weight8(w + (int64_t)(head_offset + h) * D + (c * G + gl) * 8, wv[k][c]);
      else
#pragma unroll
        for (int j = 0; j < 8; ++j) wv[k][c][j] = 0.f;
    }
  }

  int64_t i = 0;
  RingPos pos;
  for (; i < n; ++i, pos.advance(stages)) {
    const int s = pos.s;
    const bool ok = mbar_wait_bounded(&full[s], pos.phase, err, 13);
    const int64_t t = first + i * step;
    const unsigned char* xs = buf + (size_t)s * row_bytes;
    if (ok) {
#pragma unroll
      for (int k = 0; k < R; ++k) {
        if (((k * nwarp + warp) * HPW) >= head_norm) break;  // warp-uniform: the shuffles below see whole warps
        const int h = (k * nwarp + warp) * HPW + lane / G;
        const bool live = h < head_norm;
        float cur[V][8];
        double s0 = 0.0, s1 = 0.0;  // two partial sums: half the length of the dependent chain
        float amin = 1.0f;
#pragma unroll
        for (int c = 0; c < V; ++c) {
          if (live) {
            const unsigned char* src = xs + ((size_t)h * D + (c * G + gl) * 8) * sizeof(T);
            if constexpr (sizeof(T) == 4) {
              const uint4 a = lds_u4(src), b = lds_u4(src + 16);
              cur[c][0] = __uint_as_float(a.x); cur[c][1] = __uint_as_float(a.y); cur[c][2] = __uint_as_float(a.z); cur[c][3] = __uint_as_float(a.w);
              cur[c][4] = __uint_as_float(b.x); cur[c][5] = __uint_as_float(b.y); cur[c][6] = __uint_as_float(b.z); cur[c][7] = __uint_as_float(b.w);
            } else if constexpr (ElemTraits<T>::code == MCOP_BF16) {
              unpack_bf16x8(lds_u4(src), cur[c]);
            } else {
              unpack_f16x8(lds_u4(src), cur[c]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) cur[c][j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            s0 = fma((double)cur[c][j], (double)cur[c][j], s0);
            s1 = fma((double)cur[c][j + 1], (double)cur[c][j + 1], s1);
            amin = min3_abs(cur[c][j], cur[c][j + 1], amin);
          }
        }
        double ss = s0 + s1;
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (live) {
          const float var = (float)(ss * (1.0 / D));
          const float r = 1.0f / sqrtf(var + eps);
          // fast path: r within 2^-30 .. 2^30 (not a NaN) and no element of this lane below 2^-60
          const bool fast = r >= 9.31322574615478515625e-10f && r <= 1073741824.0f && amin >= 8.67361737988403547206e-19f;
          const float inv = __frcp_rn(r);
          const float2 inv2 = make_float2(inv, inv), nr2 = make_float2(-r, -r);
#pragma unroll
          for (int c = 0; c < V; ++c) {
            float o8[8];
            if (fast) {
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                const float2 a = make_float2(cur[c][j], cur[c][j + 1]);
                const float2 q0 = mul2_rn(a, inv2);
                const float2 q1 = __ffma2_rn(__ffma2_rn(q0, nr2, a), inv2, q0);
                const float2 q2 = __ffma2_rn(__ffma2_rn(q1, nr2, a), inv2, q1);
                const float2 nw = mul2_rn(q2, make_float2(wv[k][c][j], wv[k][c][j + 1]));
                o8[j] = nw.x;
                o8[j + 1] = nw.y;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) o8[j] = __fmul_rn(__fdiv_rn(cur[c][j], r), wv[k][c][j]);   // the divide-by-rsqrt convention
            }
            Vec8<T>::store(out + (t * heads + head_offset + h) * (int64_t)D + (c * G + gl) * 8, o8);
          }
        }
      }
    }
    // the barrier of the token: agrees on success and tells that every thread has left the stage buffer
    if (!__syncthreads_and(ok)) break;
    if (threadIdx.x == 0 && i + stages < n) {
      proxy_fence_before_reuse();
      issue(s, first + (i + stages) * step);
    }
  }
  if (i < n && threadIdx.x == 0) {
    // a wait ran out: drain (bounded) what is still in flight so that no copy lands after the CTA has exited
    for (int64_t k = i; k < n && k < i + stages; ++k, pos.advance(stages))
      (void)mbar_wait_bounded(&full[pos.s], pos.phase, err, 14);
  }
}

// ---------------------------------------------------------------------------------------------
// scale_dynamic_quant: y = x * smooth; scale = max|y| / 127; q = rne(y / scale).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void scale_quant_kernel(int8_t* q, float* scales, const T* x, const float* smooth, int hidden);
// the persistent, pipelined form (defined after the row-per-CTA kernels): returns 1 when the shape does not fit it
template <typename T, bool SMOOTH>
int launch_row_quant_pipe(int8_t* out, float* scales, const T* x, const float* smooth, int64_t tokens, int hidden, cudaStream_t stream);

// Eight codes clamp(rne(y / scale)) without a division per element.  d = rn(y / scale) lies between the exact products
// y * lo and y * hi, where lo = rn(inv * (1 - 2^-21)), hi = rn(inv * (1 + 2^-21)) and inv = rn(1 / scale) (each rounding
// moves a value by at most 2^-24 of itself, the margin is 2^-22).  fma(y, lo, 1.5 * 2^23) and fma(y, hi, 1.5 * 2^23) round
// those exact products to the nearest integer, ties to even, and leave it in the low mantissa bits; rounding is monotonic,
// so when both give the same integer, rne(d) is that integer.  When they differ (a tie k + 0.5 falls inside the interval,
// whose width is at most 127 * 2^-20: about one element in 16,000 of random data, more in rows of few-bit values, where
// x = max|x| / 2 gives 63.5), when y is a NaN (the comparison is unordered), and for rows whose scale is zero, infinite or
// outside [2^-100, 2^100] (`fast` false: 1 / scale overflows or loses bits), the codes come from the quotient itself.
// Two packed fused multiply-adds and a compare per pair instead of two division sequences.
//
// The quotient itself, for a vector with an undecided element: in a `fast` row all eight are formed as q0 = rn(y * inv)
// corrected twice by q + rn(y - q * scale) * inv - the first step makes q a faithful rounding of y / scale (q0 is within
// two ulps, the fused residual is exact), the second the correctly rounded one (Markstein's theorem; inv is the correctly
// rounded reciprocal and every intermediate that matters is normal: a code other than 0 means |y| >= scale / 2 >= 2^-101) -
// five packed operations per pair, no branch per element; a NaN becomes 0 as the float-to-int conversion makes it.  Rows
// outside the `fast` range take the IEEE division per element.
struct ScaleDivisor {
  float scale;
  float2 lo2, hi2, inv2, nscale2;
  bool fast;
  __device__ __forceinline__ explicit ScaleDivisor(float s) : scale(s) {
    fast = s >= 7.888609e-31f && s <= 1.2676506e30f;  // 2^-100 .. 2^100
    const float inv = __fdiv_rn(1.0f, s);
    const float lo = __fmul_rn(inv, 0.99999952316284179688f), hi = __fmul_rn(inv, 1.00000047683715820312f);  // 1 -+ 2^-21
    lo2 = make_float2(lo, lo);
    hi2 = make_float2(hi, hi);
    inv2 = make_float2(inv, inv);
    nscale2 = make_float2(-s, -s);
  }
};
__device__ __forceinline__ uint2 quant8_by_scale(const float (&y)[8], const ScaleDivisor& dv) {
  const float2 magic2 = make_float2(12582912.0f, 12582912.0f);
  uint32_t c[8];
  bool exact = !dv.fast;
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    const float2 yy = make_float2(y[j], y[j + 1]);
    const float2 a = __ffma2_rn(yy, dv.lo2, magic2), b = __ffma2_rn(yy, dv.hi2, magic2);
    exact |= (a.x != b.x) | (a.y != b.y);  // a NaN compares unequal too
    c[j] = __float_as_uint(a.x);
    c[j + 1] = __float_as_uint(a.y);
  }
  if (exact) {
    if (dv.fast) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float2 yy = make_float2(y[j], y[j + 1]);
        const float2 q0 = mul2_rn(yy, dv.inv2);
        const float2 q1 = __ffma2_rn(__ffma2_rn(q0, dv.nscale2, yy), dv.inv2, q0);
        const float2 q2 = __ffma2_rn(__ffma2_rn(q1, dv.nscale2, yy), dv.inv2, q1);
        c[j] = q2.x == q2.x ? rn_low_byte(q2.x) : 0u;          // |q| <= 127 * (1 + 2^-23): in range without a clamp
        c[j + 1] = q2.y == q2.y ? rn_low_byte(q2.y) : 0u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = (uint32_t)q_rn_clamp(__fdiv_rn(y[j], dv.scale), -128, 127);
    }
  }
  return make_uint2(pack4_low_bytes(c[0], c[1], c[2], c[3]), pack4_low_bytes(c[4], c[5], c[6], c[7]));
}

// Row in registers: x and the smooth vector are read once (the any-shape kernel below reads both twice).
// FULL: the row is exactly THREADS * NVEC vectors of 8.
template <typename T, int THREADS, int NVEC, bool FULL = false>
__global__ void __launch_bounds__(THREADS) scale_quant_vec(int8_t* q, float* scales, const T* x, const float* smooth, int hidden) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const int nv = hidden >> 3;
  const T* xr = x + row * (int64_t)hidden;
  float y[NVEC][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int k = threadIdx.x + i * THREADS;
    if (FULL || k < nv) {
      float v[8];
      Vec8<T>::load_nc(xr + k * 8, v);
      const float4 s0 = __ldg(reinterpret_cast<const float4*>(smooth + k * 8)), s1 = __ldg(reinterpret_cast<const float4*>(smooth + k * 8) + 1);
      const float sm[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        y[i][j] = __fmul_rn(v[j], sm[j]);
        amax = fmaxf(amax, fabsf(y[i][j]));
      }
    }
  }
  amax = block_reduce<true>(amax, red);
  const float scale = amax / 127.0f;
  if (threadIdx.x == 0) scales[row] = scale;
  int8_t* qr = q + row * (int64_t)hidden;
  const ScaleDivisor dv(scale);  // the contract divides by the scale
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int k = threadIdx.x + i * THREADS;
    if (FULL || k < nv) st_cs_u2(qr + k * 8, quant8_by_scale(y[i], dv));
  }
}

template <typename T>
int launch_scale_quant(int8_t* out, float* scales, const T* x, const float* smooth, int64_t tokens, int hidden, cudaStream_t s) {
  const int nv = hidden >> 3;
  const unsigned grid = (unsigned)tokens;
  {
    // measured at 65,536 x 7168 bf16: 240 us against 275 us for the row-per-CTA kernel below (random smooth scales)
    const int rc = launch_row_quant_pipe<T, true>(out, scales, x, smooth, tokens, hidden, s);
    if (rc != 1) return rc;  // 1 = not applicable: the row-per-CTA kernels below
  }
  const bool vec_ok = hidden % 8 == 0 && nv <= 4096 && aligned16(x) && aligned16(smooth) && (reinterpret_cast<uintptr_t>(out) & 7u) == 0;
  if (!vec_ok) scale_quant_kernel<T><<<grid, 256, 0, s>>>(out, scales, x, smooth, hidden);
  else if (nv <= 256) scale_quant_vec<T, 128, 2><<<grid, 128, 0, s>>>(out, scales, x, smooth, hidden);
  else if (nv == 512) scale_quant_vec<T, 128, 4, true><<<grid, 128, 0, s>>>(out, scales, x, smooth, hidden);
  else if (nv == 640) scale_quant_vec<T, 160, 4, true><<<grid, 160, 0, s>>>(out, scales, x, smooth, hidden);
  else if (nv == 768) scale_quant_vec<T, 192, 4, true><<<grid, 192, 0, s>>>(out, scales, x, smooth, hidden);
  else if (nv == 896) scale_quant_vec<T, 224, 4, true><<<grid, 224, 0, s>>>(out, scales, x, smooth, hidden);
  else if (nv <= 1024) scale_quant_vec<T, 256, 4><<<grid, 256, 0, s>>>(out, scales, x, smooth, hidden);
  else if (nv <= 2048) scale_quant_vec<T, 512, 4><<<grid, 512, 0, s>>>(out, scales, x, smooth, hidden);
  else scale_quant_vec<T, 1024, 4><<<grid, 1024, 0, s>>>(out, scales, x, smooth, hidden);
  return check_launch("scale_dynamic_quant_i8");
}
// (the any-shape kernel:)
template <typename T>
__global__ void __launch_bounds__(256) scale_quant_kernel(int8_t* q, float* scales, const T* x, const float* smooth, int hidden) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * (int64_t)hidden;
  float amax = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    amax = fmaxf(amax, fabsf(ElemTraits<T>::to_float(xr[i]) * smooth[i]));
  amax = block_reduce<true>(amax, red);
  const float scale = amax / 127.0f;
  if (threadIdx.x == 0) scales[row] = scale;
  int8_t* qr = q + row * (int64_t)hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    qr[i] = (int8_t)q_rn_clamp(ElemTraits<T>::to_float(xr[i]) * smooth[i] / scale, -128, 127);
}

// ---------------------------------------------------------------------------------------------
// dynamic_scaled_int8_quant (symmetric): scale = max|x| / 127; q = rne(x * (127 / max|x|)), 0 for an all-zero row.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) dynamic_int8_quant_kernel(int8_t* q, float* scales, const T* x, int hidden) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * (int64_t)hidden;
  float amax = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) amax = fmaxf(amax, fabsf(ElemTraits<T>::to_float(xr[i])));
  amax = block_reduce<true>(amax, red);
  if (threadIdx.x == 0) scales[row] = amax / 127.0f;
  const float inv = amax == 0.f ? 0.f : 127.0f / amax;
  int8_t* qr = q + row * (int64_t)hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    qr[i] = (int8_t)q_rn_clamp(ElemTraits<T>::to_float(xr[i]) * inv, -128, 127);
}

// the same with the row held in registers: one 16-byte (fp32: two) load per 8 elements, one 8-byte store.
// FULL: the row is exactly THREADS * NVEC vectors, so the passes need no bounds test (hidden 4096 ... 7168 with THREADS = nv / 4).
template <typename T, int THREADS, int NVEC, bool FULL = false>
__global__ void __launch_bounds__(THREADS) dynamic_int8_quant_vec(int8_t* q, float* scales, const T* x, int hidden) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const int nv = hidden >> 3;
  const T* xr = x + row * (int64_t)hidden;
  float v[NVEC][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int k = threadIdx.x + i * THREADS;
    if (FULL || k < nv) {
      Vec8<T>::load_nc(xr + k * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    }
  }
  amax = block_reduce<true>(amax, red);
  if (threadIdx.x == 0) scales[row] = amax / 127.0f;
  const float inv = amax == 0.f ? 0.f : 127.0f / amax;
  int8_t* qr = q + row * (int64_t)hidden;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int k = threadIdx.x + i * THREADS;
    if (FULL || k < nv) {
      st_cs_u2(qr + k * 8, quant8_rn_unclamped(v[i], inv));
    }
  }
}

template <typename T>
int launch_dynamic_int8_quant(int8_t* out, float* scales, const T* x, int64_t tokens, int hidden, cudaStream_t s) {
  const int nv = hidden >> 3;
  const unsigned grid = (unsigned)tokens;
  // (no pipelined form here: without a smooth vector to keep in registers the row-per-CTA kernel below, with a dozen CTAs
  // resident per SM, measured 208 us at 65,536 x 7168 bf16 against 252 us for the ring form of scale_dynamic_quant)
  const bool vec_ok = hidden % 8 == 0 && nv <= 4096 && aligned16(x) && (reinterpret_cast<uintptr_t>(out) & 7u) == 0;
  if (!vec_ok) dynamic_int8_quant_kernel<T><<<grid, 256, 0, s>>>(out, scales, x, hidden);
  else if (nv <= 256) dynamic_int8_quant_vec<T, 128, 2><<<grid, 128, 0, s>>>(out, scales, x, hidden);
  else if (nv == 512) dynamic_int8_quant_vec<T, 128, 4, true><<<grid, 128, 0, s>>>(out, scales, x, hidden);
  else if (nv == 640) dynamic_int8_quant_vec<T, 160, 4, true><<<grid, 160, 0, s>>>(out, scales, x, hidden);
  else if (nv == 768) dynamic_int8_quant_vec<T, 192, 4, true><<<grid, 192, 0, s>>>(out, scales, x, hidden);
  else if (nv == 896) dynamic_int8_quant_vec<T, 224, 4, true><<<grid, 224, 0, s>>>(out, scales, x, hidden);
  else if (nv <= 1024) dynamic_int8_quant_vec<T, 256, 4><<<grid, 256, 0, s>>>(out, scales, x, hidden);
  else if (nv <= 2048) dynamic_int8_quant_vec<T, 512, 4><<<grid, 512, 0, s>>>(out, scales, x, hidden);
  else dynamic_int8_quant_vec<T, 1024, 4><<<grid, 1024, 0, s>>>(out, scales, x, hidden);
  return check_launch("dynamic_scaled_int8_quant");
}


// ---------------------------------------------------------------------------------------------
// Persistent, pipelined form of scale_dynamic_quant for 2-byte activations: y = x * smooth; scale = max|y| / 127;
// q = clamp(rne(y / scale)).  (SMOOTH = false is the same walk for dynamic_scaled_int8_quant, scale = max|x| / 127,
// q = rne(x * (127 / max|x|)); it is not dispatched: with no smooth vector to keep the row-per-CTA kernel is faster.)
// A CTA walks the rows blockIdx.x, blockIdx.x + gridDim.x, ...; the rows `stages` ahead are on their way into shared
// memory (bulk asynchronous copies completing on an mbarrier), the smooth vector stays in registers for every row of
// the CTA (the row-per-CTA kernels fetch its 4 bytes per element again for every row: twice the row's own bytes), and
// a row costs one CTA barrier (the warps' maxima go to slots that alternate between consecutive rows).
//
// The codes come from quant8_by_scale (no division per element).
// ---------------------------------------------------------------------------------------------
template <typename T, int THREADS, int NVEC, bool FULL, bool SMOOTH>
__global__ void __launch_bounds__(THREADS, (THREADS <= 256 ? 2 : 1))
row_quant_pipe(int8_t* q, float* scales, const T* x, const float* smooth, int hidden, int64_t tokens, int stages, int* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float red[2][32];
  constexpr int NWARP = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // `stages` (<= 8) barriers in the first 128 bytes
  unsigned char* buf = smem + 128;
  const int nv = hidden >> 3;
  const uint32_t row_bytes = (uint32_t)hidden * 2u;
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t n = first < tokens ? (tokens - first + step - 1) / step : 0;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();
  pdl_wait();  // nothing of global memory is touched before the kernels ahead in the stream have completed
  auto issue = [&](int s, int64_t row) {
    mbar_expect_tx(&full[s], row_bytes);
    bulk_g2s(buf + (size_t)s * row_bytes, x + row * (int64_t)hidden, row_bytes, &full[s]);
  };
  if (threadIdx.x == 0)
    for (int s = 0; s < stages && s < n; ++s) issue(s, first + s * step);

  float sm[SMOOTH ? NVEC : 1][8];
  if constexpr (SMOOTH) {
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
      const int v = threadIdx.x + k * THREADS;
      if (FULL || v < nv) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(smooth + v * 8)), b = __ldg(reinterpret_cast<const float4*>(smooth + v * 8) + 1);
        sm[k][0] = a.x; sm[k][1] = a.y; sm[k][2] = a.z; sm[k][3] = a.w;
        sm[k][4] = b.x; sm[k][5] = b.y; sm[k][6] = b.z; sm[k][7] = b.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) sm[k][j] = 0.f;
      }
    }
  }

  int64_t i = 0;
  RingPos pos;
  uint32_t flip = 0;
  for (; i < n; ++i, pos.advance(stages), flip ^= 1u) {
    const int s = pos.s;
    const bool ok = mbar_wait_bounded(&full[s], pos.phase, err, 11);
    const int64_t row = first + i * step;
    const unsigned char* xs = buf + (size_t)s * row_bytes;
    float y[NVEC][8];
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
      const int v = threadIdx.x + k * THREADS;
      if (ok && (FULL || v < nv)) {  // when the wait ran out the stage is not read; the barrier below then ends the loop
        if (ElemTraits<T>::code == MCOP_BF16) unpack_bf16x8(lds_u4(xs + v * 16), y[k]);
        else unpack_f16x8(lds_u4(xs + v * 16), y[k]);
        if constexpr (SMOOTH) {
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const float2 pr = mul2_rn(make_float2(y[k][j], y[k][j + 1]), make_float2(sm[k][j], sm[k][j + 1]));
            y[k][j] = pr.x;
            y[k][j + 1] = pr.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; j += 2) amax = max3_abs(y[k][j], y[k][j + 1], amax);  // amax >= 0, NaNs ignored
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) y[k][j] = 0.f;
      }
    }
    amax = warp_max_nonneg(amax);
    if (lane == 0) red[flip][warp] = amax;
    // the barrier of the row: agrees on success, publishes the warps' maxima, tells that every thread has left the stage
    if (!__syncthreads_and(ok)) break;
    if (threadIdx.x == 0 && i + stages < n) {
      proxy_fence_before_reuse();
      issue(s, first + (i + stages) * step);
    }
    amax = warp_max_nonneg(lane < NWARP ? red[flip][lane] : 0.f);
    const float scale = __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) scales[row] = scale;
    int8_t* qr = q + row * (int64_t)hidden;
    if constexpr (!SMOOTH) {
      const float inv = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
#pragma unroll
      for (int k = 0; k < NVEC; ++k) {
        const int v = threadIdx.x + k * THREADS;
        if (FULL || v < nv) st_cs_u2(qr + v * 8, quant8_rn_unclamped(y[k], inv));
      }
    } else {
      const ScaleDivisor dv(scale);
#pragma unroll
      for (int k = 0; k < NVEC; ++k) {
        const int v = threadIdx.x + k * THREADS;
        if (FULL || v < nv) st_cs_u2(qr + v * 8, quant8_by_scale(y[k], dv));
      }
    }
  }
  if (i < n && threadIdx.x == 0) {
    // a wait ran out: drain (bounded) what is still in flight so that no copy lands after the CTA has exited
    for (int64_t k = i; k < n && k < i + stages; ++k, pos.advance(stages))
      (void)mbar_wait_bounded(&full[pos.s], pos.phase, err, 12);
  }
}

// Returns MCOP_OK / an error, or 1 when the shape does not fit the pipelined kernel.
template <typename T, bool SMOOTH>
int launch_row_quant_pipe(int8_t* out, float* scales, const T* x, const float* smooth, int64_t tokens, int hidden, cudaStream_t stream) {
  if constexpr (sizeof(T) != 2) {
    return 1;
  } else {
    const int nv = hidden >> 3;
    if (hidden % 8 != 0 || nv < 256 || nv > 2048 || tokens < 1024 || !aligned16(x) || (SMOOTH && !aligned16(smooth)) ||
        (reinterpret_cast<uintptr_t>(out) & 7u) != 0)
      return 1;
    const size_t row_bytes = (size_t)hidden * 2;
    int stages = (int)((64 * 1024) / row_bytes);
    stages = stages < 2 ? 2 : (stages > 4 ? 4 : stages);
    const size_t smem = 128 + (size_t)stages * row_bytes;
    const bool tiles = nv == 512 || nv == 640 || nv == 768 || nv == 896;
    const int threads = tiles ? nv / 4 : (nv <= 1024 ? 256 : 512);
    int* err = pipe_error_ptr();
    auto launch = [&](auto kernel) -> int {
      const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), 200 * 1024);
      MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "row quant: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) {
        (void)cudaGetLastError();
        per_sm = 0;
      }
      if (per_sm < 1) return 1;
      if (per_sm > 4) per_sm = 4;
      int64_t grid = (int64_t)sm_count() * per_sm;
      if (grid > tokens) grid = tokens;
      (void)launch_pdl(kernel, dim3((unsigned)grid), dim3(threads), smem, stream, out, scales, x, smooth, hidden, tokens, stages, err);
      return check_launch("row quant (pipelined)");
    };
    if (threads == 128 && tiles) return launch(row_quant_pipe<T, 128, 4, true, SMOOTH>);
    if (threads == 160 && tiles) return launch(row_quant_pipe<T, 160, 4, true, SMOOTH>);
    if (threads == 192 && tiles) return launch(row_quant_pipe<T, 192, 4, true, SMOOTH>);
    if (threads == 224 && tiles) return launch(row_quant_pipe<T, 224, 4, true, SMOOTH>);
    if (threads == 256) return launch(row_quant_pipe<T, 256, 4, false, SMOOTH>);
    return launch(row_quant_pipe<T, 512, 4, false, SMOOTH>);
  }
}

}  // namespace
}  // namespace mcop

using namespace mcop;

extern "C" int mcop_dynamic_scaled_int8_quant(int8_t* out, float* scales, const void* x, int64_t tokens, int64_t hidden,
                                              int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(out && scales && x, MCOP_ERR_ARGUMENT, "dynamic_scaled_int8_quant: null pointer");
  MCOP_REQUIRE(tokens >= 0 && tokens <= 0x7fffffffLL && hidden > 0 && hidden <= 0x7fffffff, MCOP_ERR_ARGUMENT,
               "dynamic_scaled_int8_quant: bad sizes");
  if (tokens == 0) return MCOP_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case MCOP_BF16: return launch_dynamic_int8_quant(out, scales, (const __nv_bfloat16*)x, tokens, (int)hidden, s);
    case MCOP_F16: return launch_dynamic_int8_quant(out, scales, (const __half*)x, tokens, (int)hidden, s);
    case MCOP_F32: return launch_dynamic_int8_quant(out, scales, (const float*)x, tokens, (int)hidden, s);
  }
  return set_error(MCOP_ERR_UNSUPPORTED, "dynamic_scaled_int8_quant: unknown dtype code %d", dtype);
}

extern "C" int mcop_fused_add_rmsnorm(void* x, int64_t x_row_stride, void* residual, const void* weight,
                                      int64_t tokens, int64_t hidden, float eps, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(x && residual && weight, MCOP_ERR_ARGUMENT, "fused_add_rmsnorm: null pointer");
  MCOP_REQUIRE(tokens >= 0 && hidden > 0 && hidden <= 0x7fffffff && x_row_stride >= hidden, MCOP_ERR_ARGUMENT,
               "fused_add_rmsnorm: bad sizes tokens=%lld hidden=%lld stride=%lld", (long long)tokens, (long long)hidden, (long long)x_row_stride);
  NormParams p{};
  p.x = x; p.x_stride = x_row_stride; p.weight = weight; p.residual_in = residual; p.residual_out = residual;
  p.out = x; p.out_stride = x_row_stride; p.hidden = (int)hidden; p.eps = eps;
  const bool vec = rows_vectorisable(hidden, dtype, dtype, x, x_row_stride, {residual}, {weight}, nullptr);
  return dispatch_norm<kFusedAdd>(p, tokens, vec, dtype, dtype, (cudaStream_t)stream);
}

extern "C" int mcop_add_rmsnorm_quant_i8(int8_t* out, float* scales, const void* x, int64_t x_row_stride,
                                         const void* weight, void* residual, const float* scale_ub,
                                         int64_t tokens, int64_t hidden, float eps, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(out && scales && x && weight, MCOP_ERR_ARGUMENT, "add_rmsnorm_quant_i8: null pointer");
  MCOP_REQUIRE(tokens >= 0 && hidden > 0 && hidden <= 0x7fffffff && x_row_stride >= hidden, MCOP_ERR_ARGUMENT,
               "add_rmsnorm_quant_i8: bad sizes tokens=%lld hidden=%lld stride=%lld", (long long)tokens, (long long)hidden, (long long)x_row_stride);
  NormParams p{};
  p.x = x; p.x_stride = x_row_stride; p.weight = weight; p.residual_in = residual; p.residual_out = residual;
  p.q = out; p.scales = scales; p.scale_ub = scale_ub; p.hidden = (int)hidden; p.eps = eps;
  const bool vec = rows_vectorisable(hidden, dtype, dtype, x, x_row_stride, {residual}, {weight}, out);
  return dispatch_norm<kQuant>(p, tokens, vec, dtype, dtype, (cudaStream_t)stream);
}

extern "C" int mcop_add_rmsnorm_quant_i8_norm_out(int8_t* out, void* out_norm, float* scales, const void* x, int64_t x_row_stride,
                                                  const void* weight, void* residual, const float* scale_ub, int64_t tokens,
                                                  int64_t hidden, float eps, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(out && out_norm && scales && x && weight, MCOP_ERR_ARGUMENT, "add_rmsnorm_quant_i8_norm_out: null pointer");
  MCOP_REQUIRE(tokens >= 0 && hidden > 0 && hidden <= 0x7fffffff && x_row_stride >= hidden, MCOP_ERR_ARGUMENT,
               "add_rmsnorm_quant_i8_norm_out: bad sizes tokens=%lld hidden=%lld stride=%lld", (long long)tokens, (long long)hidden,
               (long long)x_row_stride);
  NormParams p{};
  p.x = x; p.x_stride = x_row_stride; p.weight = weight; p.residual_in = residual; p.residual_out = residual;
  p.out = out_norm; p.out_stride = hidden;
  p.q = out; p.scales = scales; p.scale_ub = scale_ub; p.hidden = (int)hidden; p.eps = eps;
  const bool vec = rows_vectorisable(hidden, dtype, dtype, x, x_row_stride, {residual, out_norm}, {weight}, out);
  return dispatch_norm<kQuant>(p, tokens, vec, dtype, dtype, (cudaStream_t)stream);
}

extern "C" int mcop_rmsnorm_smooth_quant_i8(int8_t* out, float* scales, void* after_res, void* after_norm,
                                            const void* x, const void* weight, const void* smooth, const void* residual,
                                            int64_t tokens, int64_t hidden, float eps, int dtype, int wdtype,
                                            mcop_stream_t stream) {
  MCOP_REQUIRE(out && scales && after_res && after_norm && x && weight && smooth, MCOP_ERR_ARGUMENT,
               "rmsnorm_smooth_quant_i8: null pointer");
  MCOP_REQUIRE(tokens >= 0 && hidden > 0 && hidden <= 0x7fffffff, MCOP_ERR_ARGUMENT, "rmsnorm_smooth_quant_i8: bad sizes");
  NormParams p{};
  p.x = x; p.x_stride = hidden; p.weight = weight; p.smooth = smooth; p.residual_in = residual; p.residual_out = after_res;
  p.out = after_norm; p.out_stride = hidden; p.q = out; p.scales = scales; p.hidden = (int)hidden; p.eps = eps;
  const bool vec = rows_vectorisable(hidden, dtype, wdtype, x, hidden, {residual, after_res, after_norm}, {weight, smooth}, out) &&
                   (wdtype != MCOP_F32 || dtype == MCOP_F32 || hidden % 8 == 0);
  return dispatch_norm<kSmoothQuant>(p, tokens, vec, dtype, wdtype, (cudaStream_t)stream);
}

extern "C" int mcop_rmsnorm(void* out, const void* x, const void* weight, void* after_res, const void* residual,
                            int64_t tokens, int64_t hidden, float eps, int rms_div, int dtype, int wdtype,
                            mcop_stream_t stream) {
  MCOP_REQUIRE(out && x && weight, MCOP_ERR_ARGUMENT, "rmsnorm: null pointer");
  MCOP_REQUIRE((after_res == nullptr) == (residual == nullptr), MCOP_ERR_ARGUMENT,
               "rmsnorm: residual and after_res must be given together");
  MCOP_REQUIRE(tokens >= 0 && hidden > 0 && hidden <= 0x7fffffff, MCOP_ERR_ARGUMENT, "rmsnorm: bad sizes");
  NormParams p{};
  p.x = x; p.x_stride = hidden; p.weight = weight; p.residual_in = residual; p.residual_out = after_res;
  p.out = out; p.out_stride = hidden; p.hidden = (int)hidden; p.eps = eps; p.rms_div = rms_div;
  const bool vec = rows_vectorisable(hidden, dtype, wdtype, x, hidden, {residual, after_res, out}, {weight}, nullptr);
  return dispatch_norm<kPlain>(p, tokens, vec, dtype, wdtype, (cudaStream_t)stream);
}

template <typename T>
static int head_rmsnorm_wt(void* out, const void* x, const void* weight, int64_t tokens, int64_t heads, int64_t head_dim,
                           float eps, int head_offset, int head_norm, int dtype, int wdtype, cudaStream_t stream) {
  const int64_t items = tokens * head_norm;
  if (items == 0) return MCOP_OK;
  const int warps = 8;
  const int64_t blocks = (items + warps - 1) / warps;
  MCOP_REQUIRE(blocks <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "head_rmsnorm: too many rows");
  MCOP_REQUIRE(wdtype == dtype || wdtype == MCOP_F32, MCOP_ERR_UNSUPPORTED, "head_rmsnorm: weight dtype %d with activation dtype %d", wdtype, dtype);
  // heads of 64, 128 or 256 elements on 16-byte aligned buffers: vector kernel, a head on 8, 16 or 32 lanes
  if ((head_dim == 64 || head_dim == 128 || head_dim == 256) && aligned16(out) && aligned16(x) && aligned16(weight)) {
    const int G = (int)head_dim / 8, hpw = 32 / G;
    // many tokens: the pipelined kernel, if the run of heads of a token fits its ring and its rounds.  Four vectors of
    // 8 per lane when that still leaves four warps of heads per token, else one.
    if (tokens >= 1024 && head_norm > 0) {
      const size_t row_bytes = (size_t)head_norm * head_dim * sizeof(T);
      int V = 4;
      if (G % 4 != 0 || (head_norm + 32 / (G / 4) - 1) / (32 / (G / 4)) < 4) V = 1;
      const int lanes = G / V, hpw_v = 32 / lanes;
      const int witems = (head_norm + hpw_v - 1) / hpw_v;  // warp-sized groups of heads per token
      int nwarp = 0, waste = 1 << 30;
      for (int nw = 8; nw >= 4; --nw) {
        const int rounds = (witems + nw - 1) / nw;
        if (rounds <= 4 / V && rounds * nw - witems < waste) { waste = rounds * nw - witems; nwarp = nw; }
      }
      int st = (int)((64 * 1024) / row_bytes);
      if (st > 4) st = 4;
      if (nwarp && st >= 2) {
        const size_t smem = 128 + (size_t)st * row_bytes;
        auto launch_pipe = [&](auto kernel, const auto* wt) -> int {
          const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), 200 * 1024);
          MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "head_rmsnorm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
          int per_sm = 0;
          if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, nwarp * 32, smem) != cudaSuccess || per_sm < 1) {
            (void)cudaGetLastError();
            return 1;
          }
          int64_t grid = (int64_t)sm_count() * per_sm;
          if (grid > tokens) grid = tokens;
          kernel<<<(unsigned)grid, nwarp * 32, smem, stream>>>((T*)out, (const T*)x, wt, tokens, (int)heads, eps, head_offset, head_norm, st,
                                                               pipe_error_ptr());
          return check_launch("head_rmsnorm (pipelined)");
        };
        int rc = 1;
#define MCOP_HEAD_PIPE(GG, VV)                                                                                       \
  if (lanes == GG && V == VV) rc = wdtype == dtype ? launch_pipe(head_rmsnorm_pipe<T, T, GG, VV>, (const T*)weight)  \
                                                   : launch_pipe(head_rmsnorm_pipe<T, float, GG, VV>, (const float*)weight);
        MCOP_HEAD_PIPE(8, 1) MCOP_HEAD_PIPE(16, 1) MCOP_HEAD_PIPE(32, 1) MCOP_HEAD_PIPE(2, 4) MCOP_HEAD_PIPE(4, 4) MCOP_HEAD_PIPE(8, 4)
#undef MCOP_HEAD_PIPE
        if (rc != 1) return rc;  // 1 = not applicable: the grid-stride kernel below
      }
    }
    // persistent grid: every warp walks the heads with a stride of (all warps) x (heads per warp and turn); as many CTAs
    // as are resident at once, so that the grid runs as one even wave
    const int64_t need = (items + warps * hpw - 1) / (warps * hpw);
    auto launch = [&](auto kernel, const auto* wt) -> int {
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, warps * 32, 0) != cudaSuccess || per_sm < 1) {
        (void)cudaGetLastError();
        per_sm = 4;
      }
      int64_t grid = (int64_t)sm_count() * per_sm;
      if (grid > need) grid = need;
      const int64_t step = grid * warps * hpw;
      const int64_t stride_tokens = step / head_norm;
      const int stride_heads = (int)(step - stride_tokens * head_norm);
      kernel<<<(unsigned)grid, warps * 32, 0, stream>>>((T*)out, (const T*)x, wt, items, (int)heads, eps, head_offset, head_norm, stride_tokens,
                                                        stride_heads);
      return check_launch("head_rmsnorm");
    };
#define MCOP_HEAD_CASE(GG)                                                                                   \
  if (G == GG) {                                                                                              \
    if (wdtype == dtype) return launch(head_rmsnorm_vec<T, T, GG>, (const T*)weight);                         \
    return launch(head_rmsnorm_vec<T, float, GG>, (const float*)weight);                                      \
  }
    MCOP_HEAD_CASE(8) MCOP_HEAD_CASE(16) MCOP_HEAD_CASE(32)
#undef MCOP_HEAD_CASE
  }
  if (wdtype == dtype)
    head_rmsnorm_kernel<T, T><<<(unsigned)blocks, warps * 32, 0, stream>>>((T*)out, (const T*)x, (const T*)weight, tokens,
                                                                           (int)heads, (int)head_dim, eps, head_offset, head_norm);
  else if (wdtype == MCOP_F32)
    head_rmsnorm_kernel<T, float><<<(unsigned)blocks, warps * 32, 0, stream>>>((T*)out, (const T*)x, (const float*)weight, tokens,
                                                                               (int)heads, (int)head_dim, eps, head_offset, head_norm);
  else
    return set_error(MCOP_ERR_UNSUPPORTED, "head_rmsnorm: weight dtype %d with activation dtype %d", wdtype, dtype);
  return check_launch("head_rmsnorm");
}

extern "C" int mcop_head_rmsnorm(void* out, const void* x, const void* weight, int64_t tokens, int64_t heads,
                                 int64_t head_dim, float eps, int head_offset, int head_norm, int dtype, int wdtype,
                                 mcop_stream_t stream) {
  MCOP_REQUIRE(out && x && weight, MCOP_ERR_ARGUMENT, "head_rmsnorm: null pointer");
  MCOP_REQUIRE(tokens >= 0 && heads > 0 && head_dim > 0 && head_offset >= 0 && head_norm >= 0 &&
                   (int64_t)head_offset + head_norm <= heads,
               MCOP_ERR_ARGUMENT, "head_rmsnorm: bad sizes");
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case MCOP_BF16: return head_rmsnorm_wt<__nv_bfloat16>(out, x, weight, tokens, heads, head_dim, eps, head_offset, head_norm, dtype, wdtype, s);
    case MCOP_F16: return head_rmsnorm_wt<__half>(out, x, weight, tokens, heads, head_dim, eps, head_offset, head_norm, dtype, wdtype, s);
    case MCOP_F32: return head_rmsnorm_wt<float>(out, x, weight, tokens, heads, head_dim, eps, head_offset, head_norm, dtype, wdtype, s);
  }
  return set_error(MCOP_ERR_UNSUPPORTED, "head_rmsnorm: unknown dtype code %d", dtype);
}

extern "C" int mcop_scale_dynamic_quant_i8(int8_t* out, float* scales, const void* x, const float* smooth,
                                           int64_t tokens, int64_t hidden, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(out && scales && x && smooth, MCOP_ERR_ARGUMENT, "scale_dynamic_quant_i8: null pointer");
  MCOP_REQUIRE(tokens >= 0 && tokens <= 0x7fffffffLL && hidden > 0 && hidden <= 0x7fffffff, MCOP_ERR_ARGUMENT,
               "scale_dynamic_quant_i8: bad sizes");
  if (tokens == 0) return MCOP_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case MCOP_BF16: return launch_scale_quant(out, scales, (const __nv_bfloat16*)x, smooth, tokens, (int)hidden, s);
    case MCOP_F16: return launch_scale_quant(out, scales, (const __half*)x, smooth, tokens, (int)hidden, s);
    case MCOP_F32: return launch_scale_quant(out, scales, (const float*)x, smooth, tokens, (int)hidden, s);
  }
  return set_error(MCOP_ERR_UNSUPPORTED, "scale_dynamic_quant_i8: unknown dtype code %d", dtype);
}
