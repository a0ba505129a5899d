// Residual add + RMSNorm + per-token int8 quantisation with a PADDED, PACKED output row
// (mcoplib.op.fused_add_rms_norm_dynamic_per_token_quant_padding_output,
//  op/fused_add_layernorm_per_token_quant_padding_output.cu:182-416).
//
// Every token produces one byte record of pad_size 16-bit elements: bytes [0, H) the int8 codes, bytes [H, H+4) the
// fp32 scale, the rest untouched.  The reference has two arithmetic forms and picks by the row length
// (:371-394); both are reproduced:
//   form 1 (reference: hidden == 7168, kernel :182-283)  s = float(x) + float(res); res := T(s); v = s * float(w);
//          a = max|v|; r = rsqrt(mean(s^2) + eps); scale = max(a * r / 127, FLT_EPSILON); y = v * r;
//          norm := T(y); code = rne(y * (1 / scale));
//   form 2 (reference: every other length, kernel :287-340)  s as above; res := T(s); a = max|T(T(s) * w)|;
//          r from the unrounded s; scale = max(a * r / 127, FLT_EPSILON); n = T(T(float(T(s)) * r) * w);
//          code = rne(float(n) * (1 / scale)); norm := n.
// The reference's form 2 writes only the packed record and the residual; this kernel also fills the optional
// norm / codes / scales outputs when they are given.  One CTA per row, the row stays in registers.
#include <math.h>

#include "common.cuh"
#include "tma_pipe.cuh"  // ensure_dynamic_smem()

namespace mcop {
namespace {

struct PadQuantParams {
  const void* x; void* residual; const void* weight;
  int8_t* packed; int64_t packed_row_bytes;
  void* norm; int8_t* codes; float* scales;  // optional
  int hidden; float eps;
};

__device__ __forceinline__ double pq_block_sum(double v, double* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  double r = (lane < nwarp) ? red[lane] : 0.0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}

// the value whose magnitude feeds the abs-max (before the row scalar r is known)
template <typename T, int FORM> __device__ __forceinline__ float pq_amax_term(float s, float w) {
  if (FORM == 1) return s * w;
  return round_to<T>(round_to<T>(s) * w);
}
// the normalised value that is quantised (and stored as the norm output after rounding)
template <typename T, int FORM> __device__ __forceinline__ float pq_norm_value(float s, float w, float r) {
  if (FORM == 1) return (s * w) * r;
  return round_to<T>(round_to<T>(round_to<T>(s) * r) * w);
}

// FULL: the row is exactly THREADS * NVEC vectors of 8, so the unrolled passes need no bounds test
template <typename T, int FORM, int THREADS, int NVEC, bool FULL = false>
__global__ void __launch_bounds__(THREADS) pad_quant_vec(PadQuantParams p) {
  __shared__ float red[33];
  __shared__ double red64[33];
  const int64_t row = blockIdx.x;
  const int H = p.hidden, nv = H >> 3;
  const T* x = reinterpret_cast<const T*>(p.x) + row * (int64_t)H;
  T* res = reinterpret_cast<T*>(p.residual) + row * (int64_t)H;
  const T* w = reinterpret_cast<const T*>(p.weight);
  float s[NVEC][8];
  double ss = 0.0;
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (FULL || v < nv) {
      float r8[8], w8[8];
      Vec8<T>::load_nc(x + v * 8, s[i]);
      Vec8<T>::load(res + v * 8, r8);
      Vec8<T>::load_nc(w + v * 8, w8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[i][j] += r8[j];
        ss = fma((double)s[i][j], (double)s[i][j], ss);
        amax = fmaxf(amax, fabsf(pq_amax_term<T, FORM>(s[i][j], w8[j])));
      }
      Vec8<T>::store(res + v * 8, s[i]);
    }
  }
  ss = pq_block_sum(ss, red64);
  amax = block_reduce<true>(amax, red);
  const float r = 1.0f / sqrtf((float)(ss / (double)H) + p.eps);
  const float scale = fmaxf((amax * r) / 127.0f, FLT_EPSILON);
  const float inv = 1.0f / scale;
  int8_t* rec = p.packed + row * p.packed_row_bytes;
  if (threadIdx.x == 0) {
    *reinterpret_cast<float*>(rec + H) = scale;
    if (p.scales) p.scales[row] = scale;
  }
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (FULL || v < nv) {
      float w8[8], y[8];
      Vec8<T>::load_nc(w + v * 8, w8);
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        y[j] = pq_norm_value<T, FORM>(s[i][j], w8[j], r);
        c[j] = q_rn_clamp(y[j] * inv, -128, 127);
      }
      const uint2 pk = pack_i8x8(c);
      st_cs_u2(rec + v * 8, pk);
      if (p.codes) st_cs_u2(p.codes + row * (int64_t)H + v * 8, pk);
      if (p.norm) Vec8<T>::store(reinterpret_cast<T*>(p.norm) + row * (int64_t)H + v * 8, y);
    }
  }
}

// any row length that is a multiple of 4 (the packed scale needs a 4-byte boundary); the fp32 sum is parked in
// shared memory because the residual row is overwritten in place
template <typename T, int FORM>
__global__ void __launch_bounds__(256) pad_quant_any(PadQuantParams p) {
  __shared__ float red[33];
  __shared__ double red64[33];
  extern __shared__ float keep[];
  const int64_t row = blockIdx.x;
  const int H = p.hidden;
  const T* x = reinterpret_cast<const T*>(p.x) + row * (int64_t)H;
  T* res = reinterpret_cast<T*>(p.residual) + row * (int64_t)H;
  const T* w = reinterpret_cast<const T*>(p.weight);
  double ss = 0.0;
  float amax = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float s = ElemTraits<T>::to_float(x[i]) + ElemTraits<T>::to_float(res[i]);
    res[i] = ElemTraits<T>::from_float(s);
    keep[i] = s;
    ss = fma((double)s, (double)s, ss);
    amax = fmaxf(amax, fabsf(pq_amax_term<T, FORM>(s, ElemTraits<T>::to_float(w[i]))));
  }
  ss = pq_block_sum(ss, red64);
  amax = block_reduce<true>(amax, red);
  const float r = 1.0f / sqrtf((float)(ss / (double)H) + p.eps);
  const float scale = fmaxf((amax * r) / 127.0f, FLT_EPSILON);
  const float inv = 1.0f / scale;
  int8_t* rec = p.packed + row * p.packed_row_bytes;
  if (threadIdx.x == 0) {
    *reinterpret_cast<float*>(rec + H) = scale;
    if (p.scales) p.scales[row] = scale;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float y = pq_norm_value<T, FORM>(keep[i], ElemTraits<T>::to_float(w[i]), r);
    const int8_t c = (int8_t)q_rn_clamp(y * inv, -128, 127);
    rec[i] = c;
    if (p.codes) p.codes[row * (int64_t)H + i] = c;
    if (p.norm) reinterpret_cast<T*>(p.norm)[row * (int64_t)H + i] = ElemTraits<T>::from_float(y);
  }
}

template <typename T, int FORM>
int launch_pad_quant(const PadQuantParams& p, int64_t tokens, cudaStream_t s) {
  const int H = p.hidden, nv = H >> 3;
  const bool vec_ok = H % 8 == 0 && nv <= 4096 && aligned16(p.x) && aligned16(p.residual) && aligned16(p.weight) &&
                      (reinterpret_cast<uintptr_t>(p.packed) & 7u) == 0 && p.packed_row_bytes % 8 == 0 &&
                      (!p.codes || (reinterpret_cast<uintptr_t>(p.codes) & 7u) == 0) && (!p.norm || aligned16(p.norm));
  const unsigned grid = (unsigned)tokens;
  if (vec_ok) {
    if (nv <= 256) pad_quant_vec<T, FORM, 128, 2><<<grid, 128, 0, s>>>(p);
    else if (nv == 512) pad_quant_vec<T, FORM, 128, 4, true><<<grid, 128, 0, s>>>(p);
    else if (nv == 640) pad_quant_vec<T, FORM, 160, 4, true><<<grid, 160, 0, s>>>(p);
    else if (nv == 768) pad_quant_vec<T, FORM, 192, 4, true><<<grid, 192, 0, s>>>(p);
    else if (nv == 896) pad_quant_vec<T, FORM, 224, 4, true><<<grid, 224, 0, s>>>(p);
    else if (nv <= 1024) pad_quant_vec<T, FORM, 256, 4><<<grid, 256, 0, s>>>(p);
    else if (nv <= 2048) pad_quant_vec<T, FORM, 512, 4><<<grid, 512, 0, s>>>(p);
    else pad_quant_vec<T, FORM, 1024, 4><<<grid, 1024, 0, s>>>(p);
  } else {
    const size_t smem = (size_t)H * sizeof(float);
    MCOP_REQUIRE(smem <= 200 * 1024, MCOP_ERR_UNSUPPORTED, "add_rmsnorm_quant_i8_padded: hidden %d too large for the unaligned path", H);
    if (smem > 48 * 1024) {
      const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&pad_quant_any<T, FORM>), smem);
      MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "add_rmsnorm_quant_i8_padded: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    pad_quant_any<T, FORM><<<grid, 256, smem, s>>>(p);
  }
  return check_launch("add_rmsnorm_quant_i8_padded");
}

}  // namespace
}  // namespace mcop

using namespace mcop;

extern "C" int mcop_add_rmsnorm_quant_i8_padded(const void* x, void* residual, const void* weight, void* out_packed,
                                                void* out_norm, int8_t* out_codes, float* out_scales, int64_t tokens,
                                                int64_t hidden, int64_t pad_size_elems, float eps, int form, int dtype,
                                                mcop_stream_t stream) {
  MCOP_REQUIRE(x && residual && weight && out_packed, MCOP_ERR_ARGUMENT, "add_rmsnorm_quant_i8_padded: null pointer");
  MCOP_REQUIRE(tokens >= 0 && tokens <= 0x7fffffffLL && hidden > 0 && hidden <= 0x3fffffff && hidden % 4 == 0, MCOP_ERR_ARGUMENT,
               "add_rmsnorm_quant_i8_padded: bad sizes (hidden must be a multiple of 4)");
  MCOP_REQUIRE(pad_size_elems * 2 >= hidden + 4, MCOP_ERR_ARGUMENT,
               "add_rmsnorm_quant_i8_padded: a record of %lld elements cannot hold %lld codes and the scale",
               (long long)pad_size_elems, (long long)hidden);
  MCOP_REQUIRE(form >= 0 && form <= 2, MCOP_ERR_ARGUMENT, "add_rmsnorm_quant_i8_padded: form must be 0, 1 or 2");
  if (tokens == 0) return MCOP_OK;
  if (form == 0) form = hidden == 7168 ? 1 : 2;  // the reference's choice
  PadQuantParams p{x, residual, weight, reinterpret_cast<int8_t*>(out_packed), pad_size_elems * 2, out_norm, out_codes, out_scales,
                   (int)hidden, eps};
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case MCOP_BF16:
      return form == 1 ? launch_pad_quant<__nv_bfloat16, 1>(p, tokens, s) : launch_pad_quant<__nv_bfloat16, 2>(p, tokens, s);
    case MCOP_F16:
      return form == 1 ? launch_pad_quant<__half, 1>(p, tokens, s) : launch_pad_quant<__half, 2>(p, tokens, s);
  }
  return set_error(MCOP_ERR_UNSUPPORTED, "add_rmsnorm_quant_i8_padded: activation dtype %d (bf16 or f16 expected)", dtype);
}
