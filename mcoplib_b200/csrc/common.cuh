// Shared device/host helpers for the mcop_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "mcop_b200.h"

namespace mcop {

// ---------------------------------------------------------------------------------------------
// Host side: error reporting.  set_error stores a per-thread message and returns the code.
// ---------------------------------------------------------------------------------------------
int set_error(int code, const char* fmt, ...);
int check_launch(const char* what);

#define MCOP_REQUIRE(cond, code, ...)                        \
  do {                                                       \
    if (!(cond)) return ::mcop::set_error((code), __VA_ARGS__); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------------------------
// Element types.  All arithmetic is carried out on floats; `round_to<T>` reproduces a store to T
// followed by a widening load (identity for float).
// ---------------------------------------------------------------------------------------------
template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
  static constexpr int code = MCOP_F32;
  __device__ __forceinline__ static float to_float(float v) { return v; }
  __device__ __forceinline__ static float from_float(float v) { return v; }
};
template <> struct ElemTraits<__nv_bfloat16> {
  static constexpr int code = MCOP_BF16;
  __device__ __forceinline__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};
template <> struct ElemTraits<__half> {
  static constexpr int code = MCOP_F16;
  __device__ __forceinline__ static float to_float(__half v) { return __half2float(v); }
  __device__ __forceinline__ static __half from_float(float v) { return __float2half_rn(v); }
};

template <typename T> __device__ __forceinline__ float round_to(float v) {
  return ElemTraits<T>::to_float(ElemTraits<T>::from_float(v));
}

// Runtime-coded rounding (used where the element type is not a template parameter).
__device__ __forceinline__ float round_code(float v, int code) {
  if (code == MCOP_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (code == MCOP_F16) return __half2float(__float2half_rn(v));
  return v;
}

// ---------------------------------------------------------------------------------------------
// 8-element vectors: 16 bytes for 2-byte types, 32 bytes for float.  Loads use the read-only path
// unless the buffer is also written by the kernel.
// ---------------------------------------------------------------------------------------------
template <typename T> struct Vec8 {
  __device__ __forceinline__ static void load(const T* p, float (&v)[8]);
  __device__ __forceinline__ static void load_nc(const T* p, float (&v)[8]);
  __device__ __forceinline__ static void store(T* p, const float (&v)[8]);
};

__device__ __forceinline__ uint4 ld_nc_u4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
// Coherent streaming load for buffers the same kernel later overwrites in place.
__device__ __forceinline__ uint4 ld_u4(const void* p) {
  uint4 r;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p)
               : "memory");
  return r;
}
__device__ __forceinline__ void st_u4(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
// Streaming store: the line is not expected to be read again by this kernel.
__device__ __forceinline__ void st_cs_u4(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_cs_u2(void* p, uint2 v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

__device__ __forceinline__ void unpack_bf16x8(uint4 u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void unpack_f16x8(uint4 u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    float2 f = __half22float2(h);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 pack_f16x8(const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <> struct Vec8<__nv_bfloat16> {
  __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&v)[8]) { unpack_bf16x8(ld_u4(p), v); }
  __device__ __forceinline__ static void load_nc(const __nv_bfloat16* p, float (&v)[8]) { unpack_bf16x8(ld_nc_u4(p), v); }
  __device__ __forceinline__ static void store(__nv_bfloat16* p, const float (&v)[8]) { st_u4(p, pack_bf16x8(v)); }
};
template <> struct Vec8<__half> {
  __device__ __forceinline__ static void load(const __half* p, float (&v)[8]) { unpack_f16x8(ld_u4(p), v); }
  __device__ __forceinline__ static void load_nc(const __half* p, float (&v)[8]) { unpack_f16x8(ld_nc_u4(p), v); }
  __device__ __forceinline__ static void store(__half* p, const float (&v)[8]) { st_u4(p, pack_f16x8(v)); }
};
template <> struct Vec8<float> {
  __device__ __forceinline__ static void load(const float* p, float (&v)[8]) {
    uint4 a = ld_u4(p), b = ld_u4(p + 4);
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
  }
  __device__ __forceinline__ static void load_nc(const float* p, float (&v)[8]) {
    uint4 a = ld_nc_u4(p), b = ld_nc_u4(p + 4);
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
  }
  __device__ __forceinline__ static void store(float* p, const float (&v)[8]) {
    st_u4(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
    st_u4(p + 4, make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])));
  }
};

// Required alignment (bytes) of a row for the Vec8 path.
template <typename T> constexpr int vec8_align() { return sizeof(T) == 4 ? 16 : 16; }

// ---------------------------------------------------------------------------------------------
// int8 conversion: round-half-even then clamp.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int q_rn_clamp(float v, int lo, int hi) {
  int q = __float2int_rn(v);  // NaN -> 0
  return max(lo, min(hi, q));
}
// Packed fp32x2 multiply of sm_100: both lanes rounded exactly like __fmul_rn (measured bit-identical on 4M random
// pairs).  There is deliberately no packed add here: a packed add whose operand is a single-use packed product
// is merged by the assembler into one packed fused multiply-add, even with `.rn` on both (measured: 26 % of the
// results change in the last bit), which would drop an intermediate rounding the arithmetic contracts rely on.
// Sums that follow a packed product are therefore formed lane by lane with the scalar __fadd_rn.
__device__ __forceinline__ float2 mul2_rn(float2 a, float2 b) { return __fmul2_rn(a, b); }

// Conversion without the (quarter-rate) float-to-int instruction: adding 1.5 * 2^23 makes the fp32 adder round v
// to the nearest integer, ties to even, and leaves it in the low mantissa bits, so the low byte of the sum is
// the two's-complement int8 code.  Valid for |v| < 2^22; callers guarantee -128 <= v <= 127 (and no NaN).
__device__ __forceinline__ uint32_t rn_low_byte(float v) { return __float_as_uint(__fadd_rn(v, 12582912.0f)); }
// packs the low bytes of four words
__device__ __forceinline__ uint32_t pack4_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Eight codes rne(v[j] * mul) packed into 8 bytes without a float-to-int conversion (those run at a quarter of the
// rate of an add).  Requires |v[j] * mul| <= 127.5 after rounding, which abs-max scaling guarantees
// (|v * (127 / max|v|)| <= 127 * (1 + 2^-22)); finite inputs only.
__device__ __forceinline__ uint2 quant8_rn_unclamped(const float (&v)[8], float mul) {
  uint32_t c[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) c[j] = rn_low_byte(__fmul_rn(v[j], mul));
  return make_uint2(pack4_low_bytes(c[0], c[1], c[2], c[3]), pack4_low_bytes(c[4], c[5], c[6], c[7]));
}

__device__ __forceinline__ uint2 pack_i8x8(const int (&q)[8]) {
  uint32_t a = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
  uint32_t b = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
  return make_uint2(a, b);
}

// ---------------------------------------------------------------------------------------------
// Reductions.  Block reductions return the result to every thread; `red` is >= 33 floats of
// shared memory and may be reused after the call returns (a barrier closes each call).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Warp maximum of values that are >= 0 and not NaN: for those the order of the floats is the order of their bit
// patterns as unsigned integers, so one redux.sync replaces the five shuffle + max steps.
__device__ __forceinline__ float warp_max_nonneg(float v) {
  return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
}
// max(|a|, |b|, |c|) in one instruction (three-input maximum of sm_100); a NaN operand is ignored like in fmaxf.
__device__ __forceinline__ float max3_abs(float a, float b, float c) {
  float d;
  asm("max.abs.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// min(|a|, |b|, |c|) likewise.
__device__ __forceinline__ float min3_abs(float a, float b, float c) {
  float d;
  asm("min.abs.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool IS_MAX> __device__ __forceinline__ float block_reduce(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  if (nwarp == 1) return v;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nwarp) ? red[lane] : (IS_MAX ? -FLT_MAX : 0.f);
  r = IS_MAX ? warp_max(r) : warp_sum(r);
  __syncthreads();
  return r;
}

}  // namespace mcop
