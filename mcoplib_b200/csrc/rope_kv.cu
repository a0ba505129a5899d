// Part 2 of the hot path: rotary embedding on Q/K and the int8 KV-cache store.
//
// One CTA per token.  A "slice" is 8 consecutive elements of the first half of a head together with
// the 8 paired elements of the second half (NeoX pairs i, i + rot/2), so both accesses are 16-byte
// vectors and the cos/sin values a thread needs are the same for every head it touches: they are loaded
// once per token into registers.  With the fused store, the thread that rotated a K slice also
// quantises it (the bf16-ROUNDED rotated value) into the paged int8 cache, and V slices are read once
// and written once as int8: K and V never make a second trip through HBM.
#include <atomic>

#include "common.cuh"
#include "tma_pipe.cuh"

// Token count from which the persistent pipelined kernel replaces the CTA-per-token kernel.  Measured (32/8 heads of
// 128, both kernels on one box): 1024 tokens 20.3 vs 18.4 us, 2048 tokens 20.6 vs 21.1 us, 4096 tokens 24.6 vs 30.9 us,
// 8192 tokens 37.5 vs 61.0 us.
#define MCOP_ROPE_PIPE_MIN 2048

namespace mcop {
namespace {

struct RopeParams {
  // sources / destinations of the rotated heads
  const void* q_src; void* q_dst; int64_t q_stride;   // token stride, elements
  const void* k_src; void* k_dst; int64_t k_stride;
  int64_t head_stride;
  int num_heads, num_kv_heads, head_size, rot_dim;
  // cos / sin rows
  const void* cos; const void* sin; int64_t cs_row_stride;  // elements of the table type
  uint32_t sin_flip;   // 0, or 0x80000000 to rotate by the negated angle (the transposed rotation of the backward pass)
  // positions: explicit, or derived from packed sequence bounds
  const int64_t* positions;
  const int32_t* accum_q_lens; const int32_t* cache_lens; int batch;
  // fused int8 paged store (nullable)
  const void* v_src; int64_t v_stride;
  int8_t* k_cache; int8_t* v_cache;
  const int64_t* slot_mapping; const float* k_scale; const float* v_scale;
  int block_size; int64_t num_slots;
  // fused copy store (STORE 2 of the pipelined kernel): the rotated K row and the V row of token t go, in the element type, to
  // row slot_mapping[t] of k_copy / v_copy (rows of copy_stride elements, num_slots of them; a negative row id skips)
  void* k_copy; void* v_copy; int64_t copy_stride;
  // every position is checked against the rows of the cos / sin table before it becomes an address; a token whose
  // position is outside [0, max_pos) is left untouched and MCOP_DEVERR_POSITION is recorded in the error word
  int64_t max_pos; int* err;
  // fused_rope_fwd / bwd with force_bf16_attn on f16 data: the rotated heads are rounded to and stored as bf16 in the
  // same 16-bit slots (the caller then views the tensor as bf16); only the any-shape kernel takes this form
  int out_bf16;
};

__device__ __forceinline__ void report_device_error(int* err, int code) {
  if (err) atomicCAS(err, 0, code);
}

__device__ __forceinline__ int64_t token_position(const RopeParams& p, int64_t t) {
  if (p.positions) return p.positions[t];
  if (!p.accum_q_lens) return t;
  // first sequence b with accum[b+1] > t
  int lo = 0, hi = p.batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (p.accum_q_lens[mid + 1] > t) hi = mid; else lo = mid + 1;
  }
  return (int64_t)p.cache_lens[lo] + (t - p.accum_q_lens[lo]);
}

// PER_OP: arithmetic in T (a rounding after every product and after the sum); else fp32 with one rounding.
template <typename T, bool PER_OP>
__device__ __forceinline__ void rotate8(const float (&x)[8], const float (&y)[8], const float (&c)[8],
                                        const float (&s)[8], float (&xo)[8], float (&yo)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (PER_OP) {
      xo[j] = round_to<T>(__fsub_rn(round_to<T>(__fmul_rn(x[j], c[j])), round_to<T>(__fmul_rn(y[j], s[j]))));
      yo[j] = round_to<T>(__fadd_rn(round_to<T>(__fmul_rn(y[j], c[j])), round_to<T>(__fmul_rn(x[j], s[j]))));
    } else {
      xo[j] = round_to<T>(__fsub_rn(__fmul_rn(x[j], c[j]), __fmul_rn(y[j], s[j])));
      yo[j] = round_to<T>(__fadd_rn(__fmul_rn(y[j], c[j]), __fmul_rn(x[j], s[j])));
    }
  }
}

// bf16 NeoX rotation of 8 pairs in fp32 with one rounding, on packed data: the products and sums are the packed
// fp32x2 instructions of sm_100 (each lane rounded exactly like __fmul_rn / __fadd_rn; x*c - y*s is formed as
// x*c + y*(-s), which is the same value), and the results go straight to bf16 pairs.  Also returns the ROUNDED
// results widened to fp32 when `need_f32` (the fused store quantises them).
struct CosSin8 {
  float2 c[4], s[4], ns[4];
};
__device__ __forceinline__ CosSin8 make_cos_sin(const float (&c)[8], const float (&s)[8]) {
  CosSin8 r;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    r.c[q] = make_float2(c[2 * q], c[2 * q + 1]);
    r.s[q] = make_float2(s[2 * q], s[2 * q + 1]);
    r.ns[q] = make_float2(-s[2 * q], -s[2 * q + 1]);
  }
  return r;
}
__device__ __forceinline__ void rotate_bf16x8_packed(const uint4 xr, const uint4 yr, const CosSin8& cs, uint4& xo, uint4& yo) {
  const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w}, yw[4] = {yr.x, yr.y, yr.z, yr.w};
  uint32_t ox[4], oy[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 x2 = make_float2(__uint_as_float(xw[q] << 16), __uint_as_float(xw[q] & 0xffff0000u));
    const float2 y2 = make_float2(__uint_as_float(yw[q] << 16), __uint_as_float(yw[q] & 0xffff0000u));
    // products packed, sums scalar: a packed add fed by a single-use packed product is turned into a fused
    // multiply-add by the assembler (measured), which would drop the intermediate rounding; scalar add.rn is not
    const float2 xc = mul2_rn(x2, cs.c[q]), ys = mul2_rn(y2, cs.ns[q]);
    const float2 yc = mul2_rn(y2, cs.c[q]), xs = mul2_rn(x2, cs.s[q]);
    const float2 a = make_float2(__fadd_rn(xc.x, ys.x), __fadd_rn(xc.y, ys.y));
    const float2 b = make_float2(__fadd_rn(yc.x, xs.x), __fadd_rn(yc.y, xs.y));
    __nv_bfloat162 ha = __floats2bfloat162_rn(a.x, a.y), hb = __floats2bfloat162_rn(b.x, b.y);
    ox[q] = *reinterpret_cast<uint32_t*>(&ha);
    oy[q] = *reinterpret_cast<uint32_t*>(&hb);
  }
  xo = make_uint4(ox[0], ox[1], ox[2], ox[3]);
  yo = make_uint4(oy[0], oy[1], oy[2], oy[3]);
}

__device__ __forceinline__ uint2 quant8(const float (&v)[8], float inv) {
  uint32_t c[8];
  const float2 inv2 = make_float2(inv, inv);
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    const float2 pr = mul2_rn(make_float2(v[j], v[j + 1]), inv2);
    c[j] = (uint32_t)q_rn_clamp(pr.x, -127, 127);
    c[j + 1] = (uint32_t)q_rn_clamp(pr.y, -127, 127);
  }
  // the low bytes of the clamped integers are the codes: three byte permutes per four codes
  return make_uint2(pack4_low_bytes(c[0], c[1], c[2], c[3]), pack4_low_bytes(c[4], c[5], c[6], c[7]));
}

// NeoX, rot_dim == head_size, head_size % 16 == 0, all rows 16-byte aligned.
template <typename T, typename CT, bool PER_OP, bool STORE>
__global__ void __launch_bounds__(256) rope_neox_vec(RopeParams p) {
  const int64_t t = blockIdx.x;
  const int half = p.rot_dim >> 1;
  const int hv = half >> 3;                 // slices per head
  const int j = threadIdx.x % hv;           // slice index: constant per thread (blockDim % hv == 0)
  const int64_t pos = token_position(p, t);
  if (pos < 0 || pos >= p.max_pos) {  // uniform over the CTA
    if (threadIdx.x == 0) report_device_error(p.err, MCOP_DEVERR_POSITION);
    return;
  }
  float c[8], s[8];
  Vec8<CT>::load_nc(reinterpret_cast<const CT*>(p.cos) + pos * p.cs_row_stride + j * 8, c);
  Vec8<CT>::load_nc(reinterpret_cast<const CT*>(p.sin) + pos * p.cs_row_stride + j * 8, s);
  if (p.sin_flip) {
#pragma unroll
    for (int q = 0; q < 8; ++q) s[q] = __uint_as_float(__float_as_uint(s[q]) ^ p.sin_flip);
  }

  int64_t slot = -1;
  if (STORE) {
    slot = p.slot_mapping[t];
    if (slot >= p.num_slots) {  // out-of-range slots are skipped like negative ones, and reported
      if (threadIdx.x == 0) report_device_error(p.err, MCOP_DEVERR_SLOT);
      slot = -1;
    }
  }
  const int heads_per_iter = blockDim.x / hv;
  const int nqk = p.num_heads + p.num_kv_heads;
  const CosSin8 cs8 = make_cos_sin(c, s);
  for (int h = threadIdx.x / hv; h < nqk; h += heads_per_iter) {
    const bool is_k = h >= p.num_heads;
    const int hh = is_k ? h - p.num_heads : h;
    const T* src = (is_k ? reinterpret_cast<const T*>(p.k_src) + t * p.k_stride
                         : reinterpret_cast<const T*>(p.q_src) + t * p.q_stride) + hh * p.head_stride;
    T* dst = (is_k ? reinterpret_cast<T*>(p.k_dst) + t * p.k_stride
                   : reinterpret_cast<T*>(p.q_dst) + t * p.q_stride) + hh * p.head_stride;
    float x[8], y[8], xo[8], yo[8];
    if constexpr (ElemTraits<T>::code == MCOP_BF16 && !PER_OP) {
      uint4 xp, yp;
      rotate_bf16x8_packed(ld_u4(src + j * 8), ld_u4(src + half + j * 8), cs8, xp, yp);
      st_u4(dst + j * 8, xp);
      st_u4(dst + half + j * 8, yp);
      if (STORE && is_k && slot >= 0) {
        unpack_bf16x8(xp, xo);
        unpack_bf16x8(yp, yo);
      }
    } else {
      Vec8<T>::load(src + j * 8, x);
      Vec8<T>::load(src + half + j * 8, y);
      rotate8<T, PER_OP>(x, y, c, s, xo, yo);
      Vec8<T>::store(dst + j * 8, xo);
      Vec8<T>::store(dst + half + j * 8, yo);
    }
    if (STORE && is_k && slot >= 0) {
      const float inv = 1.0f / p.k_scale[hh];
      int8_t* kc = p.k_cache + (slot * p.num_kv_heads + hh) * (int64_t)p.head_size;
      st_cs_u2(kc + j * 8, quant8(xo, inv));
      st_cs_u2(kc + half + j * 8, quant8(yo, inv));
    }
  }
  if (STORE && slot >= 0) {
    // V: 16 consecutive elements per thread -> one 16-byte int8 store
    const int vper = p.head_size >> 4;
    const int nitems = p.num_kv_heads * vper;
    for (int it = threadIdx.x; it < nitems; it += blockDim.x) {
      const int hh = it / vper, e = (it % vper) * 16;
      const T* src = reinterpret_cast<const T*>(p.v_src) + t * p.v_stride + hh * (int64_t)p.head_size + e;
      float a[8], b[8];
      Vec8<T>::load_nc(src, a);
      Vec8<T>::load_nc(src + 8, b);
      const float inv = 1.0f / p.v_scale[hh];
      const uint2 qa = quant8(a, inv), qb = quant8(b, inv);
      st_cs_u4(p.v_cache + (slot * p.num_kv_heads + hh) * (int64_t)p.head_size + e, make_uint4(qa.x, qa.y, qb.x, qb.y));
    }
  }
}

// Any rot_dim <= head_size, NeoX or GPT-J pairing, any alignment.  One thread per rotated pair.
template <typename T, typename CT, bool PER_OP, bool STORE>
__global__ void __launch_bounds__(256) rope_any(RopeParams p, int is_neox) {
  const int64_t t = blockIdx.x;
  const int half = p.rot_dim >> 1;
  const int64_t pos = token_position(p, t);
  if (pos < 0 || pos >= p.max_pos) {  // uniform over the CTA
    if (threadIdx.x == 0) report_device_error(p.err, MCOP_DEVERR_POSITION);
    return;
  }
  const CT* cr = reinterpret_cast<const CT*>(p.cos) + pos * p.cs_row_stride;
  const CT* sr = reinterpret_cast<const CT*>(p.sin) + pos * p.cs_row_stride;
  int64_t slot = -1;
  if (STORE) {
    slot = p.slot_mapping[t];
    if (slot >= p.num_slots) {
      if (threadIdx.x == 0) report_device_error(p.err, MCOP_DEVERR_SLOT);
      slot = -1;
    }
  }
  const int nqk = p.num_heads + p.num_kv_heads;
  for (int i = threadIdx.x; i < nqk * half; i += blockDim.x) {
    const int h = i / half, r = i % half;
    const bool is_k = h >= p.num_heads;
    const int hh = is_k ? h - p.num_heads : h;
    const T* src = (is_k ? reinterpret_cast<const T*>(p.k_src) + t * p.k_stride
                         : reinterpret_cast<const T*>(p.q_src) + t * p.q_stride) + hh * p.head_stride;
    T* dst = (is_k ? reinterpret_cast<T*>(p.k_dst) + t * p.k_stride
                   : reinterpret_cast<T*>(p.q_dst) + t * p.q_stride) + hh * p.head_stride;
    const int xi = is_neox ? r : 2 * r, yi = is_neox ? half + r : 2 * r + 1;
    const float x = ElemTraits<T>::to_float(src[xi]), y = ElemTraits<T>::to_float(src[yi]);
    const float c = ElemTraits<CT>::to_float(cr[r]);
    const float s = __uint_as_float(__float_as_uint(ElemTraits<CT>::to_float(sr[r])) ^ p.sin_flip);
    float xo, yo;
    if (sizeof(T) == 2 && p.out_bf16) {  // fp32 arithmetic, one rounding - to bf16 instead of T
      reinterpret_cast<__nv_bfloat16*>(dst)[xi] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s)));
      reinterpret_cast<__nv_bfloat16*>(dst)[yi] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(y, c), __fmul_rn(x, s)));
      continue;
    }
    if (PER_OP) {
      xo = round_to<T>(__fsub_rn(round_to<T>(__fmul_rn(x, c)), round_to<T>(__fmul_rn(y, s))));
      yo = round_to<T>(__fadd_rn(round_to<T>(__fmul_rn(y, c)), round_to<T>(__fmul_rn(x, s))));
    } else {
      xo = round_to<T>(__fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s)));
      yo = round_to<T>(__fadd_rn(__fmul_rn(y, c), __fmul_rn(x, s)));
    }
    dst[xi] = ElemTraits<T>::from_float(xo);
    dst[yi] = ElemTraits<T>::from_float(yo);
  }
  if (STORE && slot >= 0) {
    __syncthreads();  // the rotated K of this token is re-read from global memory below
    __threadfence_block();
    const int nkv = p.num_kv_heads * p.head_size;
    for (int i = threadIdx.x; i < nkv; i += blockDim.x) {
      const int hh = i / p.head_size, e = i % p.head_size;
      const float kv = ElemTraits<T>::to_float(reinterpret_cast<const T*>(p.k_dst)[t * p.k_stride + hh * p.head_stride + e]);
      const float vv = ElemTraits<T>::to_float(reinterpret_cast<const T*>(p.v_src)[t * p.v_stride + hh * (int64_t)p.head_size + e]);
      const int64_t o = (slot * p.num_kv_heads + hh) * (int64_t)p.head_size + e;
      p.k_cache[o] = (int8_t)q_rn_clamp(__fmul_rn(kv, 1.0f / p.k_scale[hh]), -127, 127);
      p.v_cache[o] = (int8_t)q_rn_clamp(__fmul_rn(vv, 1.0f / p.v_scale[hh]), -127, 127);
    }
  }
}

inline int esize(int dtype) { return dtype == MCOP_F32 ? 4 : 2; }

#include "rope_pipe.inl"

template <typename T, typename CT, bool PER_OP, bool STORE>
int launch_rope_rows(const RopeParams& p, int64_t tokens, int is_neox, bool vec_ok, cudaStream_t stream);

template <typename T, typename CT, bool PER_OP, int STORE>
int launch_rope_t(const RopeParams& p, int64_t tokens, int is_neox, bool vec_ok, cudaStream_t stream) {
  if (tokens == 0) return MCOP_OK;
  MCOP_REQUIRE(tokens <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "rope: %lld tokens exceed the grid limit", (long long)tokens);
  if constexpr (sizeof(T) == 2) {
    // the pipelined kernel wants positions (explicit, or sequence bounds to derive them from), heads packed back to back, a
    // key tensor, and the cos / sin halves as 16-byte aligned rows: one table row cos || sin, or two tables of half rows
    // (those land side by side in the ring stage); it pays off once there are a few waves of tokens
    const bool one_row = reinterpret_cast<const char*>(p.sin) == reinterpret_cast<const char*>(p.cos) + (size_t)(p.rot_dim / 2) * sizeof(CT);
    const bool one_table = one_row && p.cs_row_stride == p.rot_dim;
    const bool two_tables = p.cs_row_stride == p.rot_dim / 2 && ((size_t)(p.rot_dim / 2) * sizeof(CT)) % 16 == 0;
    if (vec_ok && !p.sin_flip && tokens >= MCOP_ROPE_PIPE_MIN && (p.positions || p.accum_q_lens) && p.k_src && p.num_kv_heads > 0 &&
        p.head_stride == p.head_size && (one_table || two_tables)) {
      const int rc = launch_rope_pipe<T, CT, PER_OP, STORE>(p, tokens, stream);
      if (rc != 1) return rc;
    }
  }
  if constexpr (STORE == 2) {
    return 1;  // only the pipelined kernel has the copy store: the caller rotates and copies in two launches instead
  } else {
    return launch_rope_rows<T, CT, PER_OP, STORE != 0>(p, tokens, is_neox, vec_ok, stream);
  }
}

// The row-per-CTA kernels (few tokens, gathered positions, strided heads, odd shapes).
template <typename T, typename CT, bool PER_OP, bool STORE>
int launch_rope_rows(const RopeParams& p, int64_t tokens, int is_neox, bool vec_ok, cudaStream_t stream) {
  if (vec_ok) {
    const int hv = p.rot_dim >> 4;
    const int threads = hv * (256 / hv > 0 ? 256 / hv : 1);
    rope_neox_vec<T, CT, PER_OP, STORE><<<(unsigned)tokens, threads, 0, stream>>>(p);
  } else {
    rope_any<T, CT, PER_OP, STORE><<<(unsigned)tokens, 256, 0, stream>>>(p, is_neox);
  }
  return check_launch("rope");
}

// cache_dtype == dtype -> arithmetic in T unless force_fp32_math; cache fp32 -> fp32 math.
template <int STORE>
int launch_rope(const RopeParams& p, int64_t tokens, int is_neox, int dtype, int cache_dtype, bool fp32_math,
                cudaStream_t stream) {
  const int half = p.rot_dim / 2;
  bool vec_ok = is_neox && p.rot_dim == p.head_size && (half % 8 == 0) && (p.head_size % 16 == 0) && half / 8 <= 256 &&
                aligned16(p.q_src) && aligned16(p.q_dst) && (p.q_stride * esize(dtype)) % 16 == 0 &&
                (p.head_stride * esize(dtype)) % 16 == 0 && aligned16(p.cos) && aligned16(p.sin) &&
                (p.cs_row_stride * esize(cache_dtype)) % 16 == 0;
  if (p.out_bf16) vec_ok = false;
  if (p.k_src) vec_ok = vec_ok && aligned16(p.k_src) && aligned16(p.k_dst) && (p.k_stride * esize(dtype)) % 16 == 0;
  if (STORE == 1) vec_ok = vec_ok && aligned16(p.v_src) && (p.v_stride * esize(dtype)) % 16 == 0 && aligned16(p.k_cache) && aligned16(p.v_cache);
  if (STORE == 2)
    vec_ok = vec_ok && aligned16(p.v_src) && (p.v_stride * esize(dtype)) % 16 == 0 && aligned16(p.k_copy) && aligned16(p.v_copy) &&
             (p.copy_stride * esize(dtype)) % 16 == 0;
#define MCOP_ROPE_CASE(T, CT, PER)  return launch_rope_t<T, CT, PER, STORE>(p, tokens, is_neox, vec_ok, stream)
  if (cache_dtype == MCOP_F32) {
    if (dtype == MCOP_BF16) MCOP_ROPE_CASE(__nv_bfloat16, float, false);
    if (dtype == MCOP_F16) MCOP_ROPE_CASE(__half, float, false);
    if (dtype == MCOP_F32) MCOP_ROPE_CASE(float, float, false);
  } else if (cache_dtype == dtype) {
    if (fp32_math) {
      if (dtype == MCOP_BF16) MCOP_ROPE_CASE(__nv_bfloat16, __nv_bfloat16, false);
      if (dtype == MCOP_F16) MCOP_ROPE_CASE(__half, __half, false);
    } else {
      if (dtype == MCOP_BF16) MCOP_ROPE_CASE(__nv_bfloat16, __nv_bfloat16, true);
      if (dtype == MCOP_F16) MCOP_ROPE_CASE(__half, __half, true);
    }
  }
#undef MCOP_ROPE_CASE
  return set_error(MCOP_ERR_UNSUPPORTED, "rope: activation dtype %d with cos/sin dtype %d", dtype, cache_dtype);
}

// ---------------------------------------------------------------------------------------------
// Unpaged int8 store with per-(head, dim) multipliers (store_kv_cache_cuda_interface).
// ---------------------------------------------------------------------------------------------
struct KvStoreParams {
  const void* qkv; int64_t stride_token, stride_head;
  const int32_t* q_lens; const int32_t* accum; const int32_t* cache_lens; const int32_t* slot_ids;
  int8_t* k_cache; int8_t* v_cache;
  int64_t ks_slot, ks_head, ks_pos, vs_slot, vs_head, vs_pos;
  const float* k_scale; const float* v_scale;
  int batch, q_heads, kv_heads, head_dim;
  int64_t num_slots, max_len;  // extents of the cache: a slot id or a position outside them is never turned into an address
  int* err;
};

// Sequence, in-sequence index and destination of token t; false when the token belongs to no sequence or its
// destination lies outside the cache (then MCOP_DEVERR_KV_INDEX is recorded and nothing is stored).
__device__ __forceinline__ bool kv_store_locate(const KvStoreParams& p, int64_t t, int64_t& slot, int64_t& pos) {
  int lo = 0, hi = p.batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (p.accum[mid + 1] > t) hi = mid; else lo = mid + 1;
  }
  const int64_t i = t - p.accum[lo];
  if (i < 0 || i >= p.q_lens[lo]) return false;   // token outside every sequence
  pos = (int64_t)p.cache_lens[lo] + i;
  slot = p.slot_ids[lo];
  if (slot < 0 || slot >= p.num_slots || pos < 0 || pos >= p.max_len) {
    if (threadIdx.x == 0) report_device_error(p.err, MCOP_DEVERR_KV_INDEX);
    return false;
  }
  return true;
}

// One CTA per token, one element per thread and step (any head size, any alignment).
template <typename T>
__global__ void __launch_bounds__(256) kv_store_kernel(KvStoreParams p) {
  const int64_t t = blockIdx.x;
  int64_t slot, pos;
  if (!kv_store_locate(p, t, slot, pos)) return;
  const T* tok = reinterpret_cast<const T*>(p.qkv) + t * p.stride_token;
  const int n = p.kv_heads * p.head_dim;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const int h = e / p.head_dim, d = e % p.head_dim;
    const float kv = ElemTraits<T>::to_float(tok[(p.q_heads + h) * p.stride_head + d]);
    const float vv = ElemTraits<T>::to_float(tok[(p.q_heads + p.kv_heads + h) * p.stride_head + d]);
    p.k_cache[slot * p.ks_slot + h * p.ks_head + pos * p.ks_pos + d] =
        (int8_t)q_rn_clamp(__fmul_rn(kv, p.k_scale[h * p.head_dim + d]), -127, 127);
    p.v_cache[slot * p.vs_slot + h * p.vs_head + pos * p.vs_pos + d] =
        (int8_t)q_rn_clamp(__fmul_rn(vv, p.v_scale[h * p.head_dim + d]), -127, 127);
  }
}

// Vector form: a thread takes 16 consecutive elements of one K or V head of U consecutive tokens.  The four 16-byte
// loads of the fp32 multipliers (which depend on head and element only) are made once for the U tokens, the 2 * U
// 16-byte loads of the activations are all issued before the first conversion - one token per thread left a single
// pair of loads in flight per thread behind a dependent chain of four index loads (3.7 TB/s) - and the token's
// sequence is searched once per group: the tokens after the first step forward from the first one's sequence.
// TPB token groups per CTA so that small head counts still fill the CTA.  Needs head_dim % 16 == 0 and 16-byte aligned
// rows on both sides.
template <typename T, int U>
__global__ void __launch_bounds__(256) kv_store_vec(KvStoreParams p, int64_t tokens, int groups_per_cta) {
  const int per_head = p.head_dim >> 4;
  const int per_token = 2 * p.kv_heads * per_head;   // K items, then V items
  const int gl = threadIdx.x / per_token;
  const int64_t t0 = ((int64_t)blockIdx.x * groups_per_cta + gl) * U;
  if (gl >= groups_per_cta || t0 >= tokens) return;
  const int it = threadIdx.x % per_token;
  const bool is_v = it >= p.kv_heads * per_head;
  const int r = is_v ? it - p.kv_heads * per_head : it;
  const int h = r / per_head, d = (r % per_head) * 16;

  // sequence of the first token (all threads of the group run the search: same addresses, one broadcast load each)
  int lo = 0, hi = p.batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (p.accum[mid + 1] > t0) hi = mid; else lo = mid + 1;
  }
  int8_t* dst[U];
  uint4 ra[U], rb[U];  // the raw 16-byte vectors: unpacked only when they are used
  // what does not depend on the token: this thread's place inside a token's packed row and inside a cache row
  int8_t* const cache_hd = (is_v ? p.v_cache + h * p.vs_head : p.k_cache + h * p.ks_head) + d;
  const int64_t c_slot = is_v ? p.vs_slot : p.ks_slot, c_pos = is_v ? p.vs_pos : p.ks_pos;
  const T* const src_hd = reinterpret_cast<const T*>(p.qkv) + (p.q_heads + (is_v ? p.kv_heads : 0) + h) * p.stride_head + d;
  // sequence data of the token before (most groups of U tokens lie inside one sequence: its bounds are read once)
  int cur = -1;
  int64_t seq_begin = 0, seq_len = 0, seq_cache = 0, seq_slot = -1;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t t = t0 + u;
    dst[u] = nullptr;
    if (t >= tokens) continue;
    while (lo < p.batch - 1 && p.accum[lo + 1] <= t) ++lo;  // at most `batch` steps over the whole group
    if (lo != cur) {
      cur = lo;
      seq_begin = p.accum[lo]; seq_len = p.q_lens[lo]; seq_cache = p.cache_lens[lo]; seq_slot = p.slot_ids[lo];
    }
    const int64_t i = t - seq_begin;
    if (i < 0 || i >= seq_len) continue;                     // token outside every sequence
    const int64_t pos = seq_cache + i;
    if (seq_slot < 0 || seq_slot >= p.num_slots || pos < 0 || pos >= p.max_len) {  // never becomes an address
      if (it == 0) report_device_error(p.err, MCOP_DEVERR_KV_INDEX);
      continue;
    }
    dst[u] = cache_hd + seq_slot * c_slot + pos * c_pos;
    const T* src = src_hd + t * p.stride_token;
    ra[u] = ld_nc_u4(src);
    rb[u] = ld_nc_u4(src + 8);
  }
  const float* sc = (is_v ? p.v_scale : p.k_scale) + h * p.head_dim + d;
  const float4 s0 = __ldg(reinterpret_cast<const float4*>(sc)), s1 = __ldg(reinterpret_cast<const float4*>(sc) + 1);
  const float4 s2 = __ldg(reinterpret_cast<const float4*>(sc) + 2), s3 = __ldg(reinterpret_cast<const float4*>(sc) + 3);
  const float m[16] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w, s2.x, s2.y, s2.z, s2.w, s3.x, s3.y, s3.z, s3.w};
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (!dst[u]) continue;
    float a[8], b[8];
    if (ElemTraits<T>::code == MCOP_BF16) { unpack_bf16x8(ra[u], a); unpack_bf16x8(rb[u], b); }
    else { unpack_f16x8(ra[u], a); unpack_f16x8(rb[u], b); }
    // (clamping and rounding with the fp32 adder instead of the float-to-int conversion measured slower here: 99 against
    // 90 us at 65,536 tokens of 8 + 8 heads - the NaN test it needs costs more than the conversion unit saves; packed
    // products and byte permutes instead of shifts and ors: 90 -> 84 us)
    uint32_t c[16];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const float2 pa = mul2_rn(make_float2(a[j], a[j + 1]), make_float2(m[j], m[j + 1]));
      const float2 pb = mul2_rn(make_float2(b[j], b[j + 1]), make_float2(m[8 + j], m[9 + j]));
      c[j] = (uint32_t)q_rn_clamp(pa.x, -127, 127);
      c[j + 1] = (uint32_t)q_rn_clamp(pa.y, -127, 127);
      c[8 + j] = (uint32_t)q_rn_clamp(pb.x, -127, 127);
      c[9 + j] = (uint32_t)q_rn_clamp(pb.y, -127, 127);
    }
    // the low bytes of the clamped integers are the codes: three byte permutes per four codes
    st_cs_u4(dst[u], make_uint4(pack4_low_bytes(c[0], c[1], c[2], c[3]), pack4_low_bytes(c[4], c[5], c[6], c[7]),
                                pack4_low_bytes(c[8], c[9], c[10], c[11]), pack4_low_bytes(c[12], c[13], c[14], c[15])));
  }
}

// ---------------------------------------------------------------------------------------------
// Paged copies with kv_cache_dtype "auto": reshape_and_cache_flash ([blocks, block_size, heads, head_size] by strides)
// and reshape_and_cache (K as [blocks, heads, head_size / x, block_size, x], V as [blocks, heads, head_size, block_size]).
// A negative slot is the caller's "no store" mark; a slot past the cache is skipped and reported (MCOP_DEVERR_SLOT).
// ---------------------------------------------------------------------------------------------
struct CacheCopyParams {
  const char* key; const char* value; int64_t key_stride, value_stride;   // bytes
  char* key_cache; char* value_cache; int64_t block_stride, page_stride, head_stride;  // bytes
  const int64_t* slot_mapping; int kv_heads, head_bytes, block_size;
  int64_t num_slots; int* err;
};

template <typename V>
__global__ void __launch_bounds__(256) cache_copy_kernel(CacheCopyParams p) {
  const int64_t t = blockIdx.x;
  const int64_t slot = p.slot_mapping[t];
  if (slot < 0) return;
  if (slot >= p.num_slots) {
    if (threadIdx.x == 0) report_device_error(p.err, MCOP_DEVERR_SLOT);
    return;
  }
  const int64_t blk = slot / p.block_size, off = slot % p.block_size;
  const int per_head = p.head_bytes / (int)sizeof(V);
  const int n = p.kv_heads * per_head;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int h = i / per_head, e = i % per_head;
    const int64_t dst = blk * p.block_stride + off * p.page_stride + h * p.head_stride + (int64_t)e * sizeof(V);
    const int64_t src = (int64_t)h * p.head_bytes + (int64_t)e * sizeof(V);
    *reinterpret_cast<V*>(p.key_cache + dst) = *reinterpret_cast<const V*>(p.key + t * p.key_stride + src);
    *reinterpret_cast<V*>(p.value_cache + dst) = *reinterpret_cast<const V*>(p.value + t * p.value_stride + src);
  }
}

// The same with 16-byte vectors and U tokens per thread: a thread moves one vector of K and one of V for each of its U
// tokens, all 2 * U loads issued before the first store (one token per CTA left one pair of loads per thread in flight
// behind the slot lookup: 4.7 TB/s at 8 heads of 128).  The CTA's threads are (tokens per pass) x (vectors per token).
template <int U>
__global__ void __launch_bounds__(256) cache_copy_vec16_multi(CacheCopyParams p, int64_t tokens, int tokens_per_pass) {
  const int per_head = p.head_bytes >> 4;
  const int n = p.kv_heads * per_head;
  const int tl = threadIdx.x / n, i = threadIdx.x - tl * n;
  if (tl >= tokens_per_pass) return;
  const int h = i / per_head, e = i - h * per_head;
  const int64_t src = (int64_t)h * p.head_bytes + (int64_t)e * 16;
  const int64_t dst_hd = h * p.head_stride + (int64_t)e * 16;
  const int64_t t0 = (int64_t)blockIdx.x * tokens_per_pass * U + tl;
  uint4 kv[U], vv[U];
  int64_t dst[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t t = t0 + (int64_t)u * tokens_per_pass;
    dst[u] = -1;
    if (t >= tokens) continue;
    const int64_t slot = p.slot_mapping[t];
    if (slot < 0) continue;
    if (slot >= p.num_slots) {  // never becomes an address
      if (i == 0) report_device_error(p.err, MCOP_DEVERR_SLOT);
      continue;
    }
    const int64_t blk = slot / p.block_size, off = slot % p.block_size;
    dst[u] = blk * p.block_stride + off * p.page_stride + dst_hd;
    kv[u] = ld_nc_u4(p.key + t * p.key_stride + src);
    vv[u] = ld_nc_u4(p.value + t * p.value_stride + src);
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (dst[u] < 0) continue;
    st_u4(p.key_cache + dst[u], kv[u]);
    st_u4(p.value_cache + dst[u], vv[u]);
  }
}

struct CacheSplitParams {
  const void* key; const void* value; int64_t key_stride, value_stride;  // elements
  void* key_cache; void* value_cache;
  const int64_t* slot_mapping; int kv_heads, head_size, block_size, x;
  int64_t num_slots; int* err;
};

// One CTA per token; a work item is one group of x consecutive elements of one head: the K group stays together
// (x elements at [.., head, group, offset, :]), the V elements go x rows of block_size apart.
template <typename E, typename KV>  // element, and the vector type one K group is moved as (sizeof(KV) == x * sizeof(E)), or E itself
__global__ void __launch_bounds__(256) cache_split_kernel(CacheSplitParams p) {
  const int64_t t = blockIdx.x;
  const int64_t slot = p.slot_mapping[t];
  if (slot < 0) return;
  if (slot >= p.num_slots) {
    if (threadIdx.x == 0) report_device_error(p.err, MCOP_DEVERR_SLOT);
    return;
  }
  const int64_t blk = slot / p.block_size, off = slot % p.block_size;
  const int groups = p.head_size / p.x;
  const int n = p.kv_heads * groups;
  const E* key = reinterpret_cast<const E*>(p.key) + t * p.key_stride;
  const E* value = reinterpret_cast<const E*>(p.value) + t * p.value_stride;
  E* kc = reinterpret_cast<E*>(p.key_cache);
  E* vc = reinterpret_cast<E*>(p.value_cache);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int h = i / groups, g = i % groups;
    const int64_t src = (int64_t)h * p.head_size + (int64_t)g * p.x;
    const int64_t kdst = (((blk * p.kv_heads + h) * groups + g) * p.block_size + off) * p.x;
    const int64_t vdst = ((blk * p.kv_heads + h) * (int64_t)p.head_size + (int64_t)g * p.x) * p.block_size + off;
    if (sizeof(KV) > sizeof(E)) {
      *reinterpret_cast<KV*>(kc + kdst) = *reinterpret_cast<const KV*>(key + src);
    } else {
      for (int j = 0; j < p.x; ++j) kc[kdst + j] = key[src + j];
    }
    for (int j = 0; j < p.x; ++j) vc[vdst + (int64_t)j * p.block_size] = value[src + j];
  }
}

// The same for 2-byte elements with a window of kSplitWindow consecutive tokens per CTA.  In the V layout
// [blocks, heads, head_size, block_size] the elements of one token lie block_size elements apart: written token by token
// every element is a 2-byte store into a 32-byte sector of its own (1024 partial-sector writes per token of 8 heads of
// 128: 0.9 TB/s with consecutive slots, 0.46 TB/s with scattered ones).  Tokens that follow each other in a prefill
// mostly have consecutive slots, i.e. consecutive positions of one block, and then the 2-byte pieces of neighbouring
// tokens are neighbours in memory.  So the CTA copies the V rows of its window into shared memory, splits the window
// into runs of tokens with consecutive slots inside one block, and every thread writes, for its (head, element) pairs,
// the run's values as the largest aligned pieces (16, 8, 4, 2 bytes) - a full run of 16 tokens is two 16-byte stores
// per pair instead of sixteen 2-byte stores.  K moves as before (a group of x elements per store).
constexpr int kSplitWindow = 16;

template <typename KV>
__global__ void __launch_bounds__(256) cache_split_tile_kernel(CacheSplitParams p, int64_t tokens) {
  extern __shared__ __align__(16) unsigned char tile_raw[];
  uint16_t* tile = reinterpret_cast<uint16_t*>(tile_raw);  // [kSplitWindow][kv_heads * head_size]
  __shared__ int64_t s_slot[kSplitWindow];
  const int HD = p.kv_heads * p.head_size;
  const int64_t t0 = (int64_t)blockIdx.x * kSplitWindow;
  const int nt = (int)min((int64_t)kSplitWindow, tokens - t0);
  if (threadIdx.x < kSplitWindow) {
    int64_t slot = -1;
    if (threadIdx.x < nt) {
      slot = p.slot_mapping[t0 + threadIdx.x];
      if (slot >= p.num_slots) {  // never becomes an address
        report_device_error(p.err, MCOP_DEVERR_SLOT);
        slot = -1;
      }
    }
    s_slot[threadIdx.x] = slot;
  }
  // V rows of the window -> shared memory, 16 bytes at a time (rows of HD elements, HD % 8 == 0)
  const uint16_t* value = reinterpret_cast<const uint16_t*>(p.value);
  const int vec_per_row = HD >> 3;
  for (int i = threadIdx.x; i < nt * vec_per_row; i += blockDim.x) {
    const int tk = i / vec_per_row, v = i - tk * vec_per_row;
    *reinterpret_cast<uint4*>(tile + (size_t)tk * HD + v * 8) = ld_nc_u4(value + (t0 + tk) * p.value_stride + v * 8);
  }
  __syncthreads();
  // K: one group of x elements per store, token by token
  {
    const int groups = p.head_size / p.x;
    const int n = p.kv_heads * groups;
    const uint16_t* key = reinterpret_cast<const uint16_t*>(p.key);
    uint16_t* kc = reinterpret_cast<uint16_t*>(p.key_cache);
    // consecutive lanes take consecutive TOKENS of one group: with consecutive slots their 16-byte groups are neighbours
    // in the cache (a whole 256-byte line of one (head, group) per 16 lanes) instead of 32 half-written sectors: 142 -> 128 us at
    // 65,536 tokens of 8 heads of 128 (the K rows through shared memory as well: 157 us)
    for (int i = threadIdx.x; i < nt * n; i += blockDim.x) {
      const int r = i / nt, tk = i - r * nt;
      const int64_t slot = s_slot[tk];
      if (slot < 0) continue;
      const int64_t blk = slot / p.block_size, off = slot % p.block_size;
      const int h = r / groups, g = r - h * groups;
      const int64_t src = (t0 + tk) * p.key_stride + (int64_t)h * p.head_size + (int64_t)g * p.x;
      const int64_t kdst = (((blk * p.kv_heads + h) * groups + g) * p.block_size + off) * p.x;
      if (sizeof(KV) > sizeof(uint16_t)) {
        *reinterpret_cast<KV*>(kc + kdst) = *reinterpret_cast<const KV*>(key + src);
      } else {
        for (int j = 0; j < p.x; ++j) kc[kdst + j] = key[src + j];
      }
    }
  }
  // V: runs of tokens with consecutive slots inside one block
  uint16_t* vc = reinterpret_cast<uint16_t*>(p.value_cache);
  int a = 0;
  while (a < nt) {  // the same for every thread of the CTA
    const int64_t slot0 = s_slot[a];
    if (slot0 < 0) { ++a; continue; }
    const int64_t blk = slot0 / p.block_size;
    const int off0 = (int)(slot0 % p.block_size);
    int n = 1;
    while (a + n < nt && s_slot[a + n] == slot0 + n && off0 + n < p.block_size) ++n;
    for (int hd = threadIdx.x; hd < HD; hd += blockDim.x) {
      const int h = hd / p.head_size, d = hd - h * p.head_size;
      uint16_t* dst = vc + ((blk * p.kv_heads + h) * (int64_t)p.head_size + d) * p.block_size + off0;
      const uint16_t* col = tile + (size_t)a * HD + hd;  // the run's values: col[i * HD]
      int i = 0;
      while (i < n) {
        const uintptr_t addr = reinterpret_cast<uintptr_t>(dst + i);
        const int left = n - i;
        if (left >= 8 && (addr & 15u) == 0) {
          uint32_t w[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) w[q] = (uint32_t)col[(size_t)(i + 2 * q) * HD] | ((uint32_t)col[(size_t)(i + 2 * q + 1) * HD] << 16);
          *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
          i += 8;
        } else if (left >= 4 && (addr & 7u) == 0) {
          uint32_t w[2];
#pragma unroll
          for (int q = 0; q < 2; ++q) w[q] = (uint32_t)col[(size_t)(i + 2 * q) * HD] | ((uint32_t)col[(size_t)(i + 2 * q + 1) * HD] << 16);
          *reinterpret_cast<uint2*>(dst + i) = make_uint2(w[0], w[1]);
          i += 4;
        } else if (left >= 2 && (addr & 3u) == 0) {
          *reinterpret_cast<uint32_t*>(dst + i) = (uint32_t)col[(size_t)i * HD] | ((uint32_t)col[(size_t)(i + 1) * HD] << 16);
          i += 2;
        } else {
          dst[i] = col[(size_t)i * HD];
          i += 1;
        }
      }
    }
    a += n;
  }
}

}  // namespace
}  // namespace mcop

using namespace mcop;

extern "C" int mcop_rope_inplace(const int64_t* positions, void* query, void* key, const void* cos_sin_cache,
                                 int cache_dtype, int64_t max_position, int64_t tokens, int num_heads, int num_kv_heads,
                                 int head_size, int rot_dim, int64_t query_stride, int64_t key_stride, int64_t head_stride,
                                 int is_neox, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(positions && query && cos_sin_cache, MCOP_ERR_ARGUMENT, "rope_inplace: null pointer");
  MCOP_REQUIRE(tokens >= 0 && num_heads > 0 && num_kv_heads >= 0 && head_size > 0 && rot_dim > 0 && rot_dim % 2 == 0 &&
                   rot_dim <= head_size && max_position > 0, MCOP_ERR_ARGUMENT, "rope_inplace: bad sizes");
  RopeParams p{};
  p.q_src = query; p.q_dst = query; p.q_stride = query_stride;
  p.k_src = key; p.k_dst = key; p.k_stride = key_stride; p.head_stride = head_stride;
  p.num_heads = num_heads; p.num_kv_heads = key ? num_kv_heads : 0; p.head_size = head_size; p.rot_dim = rot_dim;
  const int cs = cache_dtype == MCOP_F32 ? 4 : 2;
  p.cos = cos_sin_cache; p.sin = reinterpret_cast<const char*>(cos_sin_cache) + (size_t)(rot_dim / 2) * cs;
  p.cs_row_stride = rot_dim; p.positions = positions;
  p.max_pos = max_position; p.err = pipe_error_ptr();
  return launch_rope<0>(p, tokens, is_neox, dtype, cache_dtype, false, (cudaStream_t)stream);
}

extern "C" int mcop_rope_packed(const void* packed_qkv, void* output, const float* cos, const float* sin, int64_t max_position,
                                const int32_t* accum_q_lens, const int32_t* cache_lens, int batch, int64_t tokens,
                                int q_heads, int kv_heads, int head_dim, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(packed_qkv && output && cos && sin && accum_q_lens && cache_lens, MCOP_ERR_ARGUMENT, "rope_packed: null pointer");
  MCOP_REQUIRE(tokens >= 0 && batch > 0 && q_heads > 0 && kv_heads >= 0 && head_dim > 0 && head_dim % 2 == 0 && max_position > 0,
               MCOP_ERR_ARGUMENT, "rope_packed: bad sizes");
  const int64_t tok_stride = (int64_t)(q_heads + 2 * kv_heads) * head_dim;
  const int es = dtype == MCOP_F32 ? 4 : 2;
  RopeParams p{};
  p.q_src = packed_qkv; p.q_dst = output; p.q_stride = tok_stride;
  p.k_src = reinterpret_cast<const char*>(packed_qkv) + (size_t)q_heads * head_dim * es;
  p.k_dst = reinterpret_cast<char*>(output) + (size_t)q_heads * head_dim * es;
  p.k_stride = tok_stride; p.head_stride = head_dim;
  p.num_heads = q_heads; p.num_kv_heads = kv_heads; p.head_size = head_dim; p.rot_dim = head_dim;
  p.cos = cos; p.sin = sin; p.cs_row_stride = head_dim / 2;
  p.accum_q_lens = accum_q_lens; p.cache_lens = cache_lens; p.batch = batch;
  p.max_pos = max_position; p.err = pipe_error_ptr();
  return launch_rope<0>(p, tokens, 1, dtype, MCOP_F32, true, (cudaStream_t)stream);
}

static int fused_rope_planes(const char* name, void* qkv, const void* cos, const void* sin, int64_t max_position, const int64_t* indexes,
                             int64_t seq, int planes, int heads, int head_dim, int dtype, int out_bf16, uint32_t sin_flip,
                             mcop_stream_t stream) {
  MCOP_REQUIRE(qkv && cos && sin, MCOP_ERR_ARGUMENT, "%s: null pointer", name);
  MCOP_REQUIRE(seq >= 0 && planes >= 2 && heads > 0 && head_dim > 0 && head_dim % 2 == 0 && max_position > 0, MCOP_ERR_ARGUMENT,
               "%s: bad sizes", name);
  MCOP_REQUIRE(dtype == MCOP_BF16 || dtype == MCOP_F16, MCOP_ERR_UNSUPPORTED, "%s: only f16 and bf16", name);
  MCOP_REQUIRE(!out_bf16 || dtype == MCOP_F16, MCOP_ERR_ARGUMENT, "%s: the bf16 output form applies to f16 data only", name);
  const int64_t tok_stride = (int64_t)planes * heads * head_dim;
  RopeParams p{};
  p.q_src = qkv; p.q_dst = qkv; p.q_stride = tok_stride;
  p.k_src = reinterpret_cast<char*>(qkv) + (size_t)heads * head_dim * 2;
  p.k_dst = reinterpret_cast<char*>(qkv) + (size_t)heads * head_dim * 2;
  p.k_stride = tok_stride; p.head_stride = head_dim;
  p.num_heads = heads; p.num_kv_heads = heads; p.head_size = head_dim; p.rot_dim = head_dim;
  p.cos = cos; p.sin = sin; p.cs_row_stride = head_dim / 2; p.positions = indexes;
  p.sin_flip = sin_flip;
  p.out_bf16 = out_bf16 ? 1 : 0;
  p.max_pos = max_position; p.err = pipe_error_ptr();
  return launch_rope<0>(p, seq, 1, dtype, dtype, true, (cudaStream_t)stream);
}

extern "C" int mcop_fused_rope_fwd(void* qkv, const void* cos, const void* sin, int64_t max_position, const int64_t* indexes,
                                   int64_t seq, int planes, int heads, int head_dim, int dtype, int out_bf16, mcop_stream_t stream) {
  return fused_rope_planes("fused_rope_fwd", qkv, cos, sin, max_position, indexes, seq, planes, heads, head_dim, dtype, out_bf16, 0u,
                           stream);
}

// x' = x*c + y*s, y' = y*c - x*s: the forward rotation with the sine negated (negation is exact, so every product
// and sum rounds as in the forward form).
extern "C" int mcop_fused_rope_bwd(void* qkv, const void* cos, const void* sin, int64_t max_position, const int64_t* indexes,
                                   int64_t seq, int planes, int heads, int head_dim, int dtype, int out_bf16, mcop_stream_t stream) {
  return fused_rope_planes("fused_rope_bwd", qkv, cos, sin, max_position, indexes, seq, planes, heads, head_dim, dtype, out_bf16,
                           0x80000000u, stream);
}

extern "C" int mcop_rope_kv_store_i8_paged(const int64_t* positions, void* query, void* key, const void* value,
                                           const void* cos_sin_cache, int cache_dtype, int64_t max_position, int8_t* key_cache,
                                           int8_t* value_cache, const int64_t* slot_mapping, const float* k_scale,
                                           const float* v_scale, int64_t tokens, int num_heads, int num_kv_heads,
                                           int head_size, int rot_dim, int64_t query_stride, int64_t key_stride,
                                           int64_t value_stride, int block_size, int64_t num_blocks, int is_neox,
                                           int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(positions && query && key && value && cos_sin_cache && key_cache && value_cache && slot_mapping && k_scale && v_scale,
               MCOP_ERR_ARGUMENT, "rope_kv_store_i8_paged: null pointer");
  MCOP_REQUIRE(tokens >= 0 && num_heads > 0 && num_kv_heads > 0 && head_size > 0 && rot_dim > 0 && rot_dim % 2 == 0 &&
                   rot_dim <= head_size && block_size > 0 && num_blocks >= 0 && max_position > 0,
               MCOP_ERR_ARGUMENT, "rope_kv_store_i8_paged: bad sizes");
  RopeParams p{};
  p.q_src = query; p.q_dst = query; p.q_stride = query_stride;
  p.k_src = key; p.k_dst = key; p.k_stride = key_stride; p.head_stride = head_size;
  p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.head_size = head_size; p.rot_dim = rot_dim;
  const int cs = cache_dtype == MCOP_F32 ? 4 : 2;
  p.cos = cos_sin_cache; p.sin = reinterpret_cast<const char*>(cos_sin_cache) + (size_t)(rot_dim / 2) * cs;
  p.cs_row_stride = rot_dim; p.positions = positions;
  p.v_src = value; p.v_stride = value_stride; p.k_cache = key_cache; p.v_cache = value_cache;
  p.slot_mapping = slot_mapping; p.k_scale = k_scale; p.v_scale = v_scale;
  p.block_size = block_size; p.num_slots = num_blocks * block_size;
  p.max_pos = max_position; p.err = pipe_error_ptr();
  return launch_rope<1>(p, tokens, is_neox, dtype, cache_dtype, false, (cudaStream_t)stream);
}

extern "C" int mcop_rope_kv_copy(const int64_t* positions, void* query, void* key, const void* value, const float* cos_sin_cache,
                                 int64_t max_position, void* k_buffer, void* v_buffer, const int64_t* kv_loc, int64_t buffer_rows,
                                 int64_t buffer_row_stride, int64_t tokens, int num_heads, int num_kv_heads, int head_size,
                                 int64_t query_stride, int64_t key_stride, int64_t value_stride, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(positions && query && key && value && cos_sin_cache && k_buffer && v_buffer && kv_loc, MCOP_ERR_ARGUMENT,
               "rope_kv_copy: null pointer");
  MCOP_REQUIRE(tokens >= 0 && num_heads > 0 && num_kv_heads > 0 && head_size > 0 && head_size % 2 == 0 && max_position > 0 &&
                   buffer_rows >= 0 && buffer_row_stride >= (int64_t)num_kv_heads * head_size,
               MCOP_ERR_ARGUMENT, "rope_kv_copy: bad sizes");
  MCOP_REQUIRE(dtype == MCOP_BF16 || dtype == MCOP_F16, MCOP_ERR_UNSUPPORTED, "rope_kv_copy: only f16 and bf16");
  if (tokens == 0) return MCOP_OK;
  RopeParams p{};
  p.q_src = query; p.q_dst = query; p.q_stride = query_stride;
  p.k_src = key; p.k_dst = key; p.k_stride = key_stride; p.head_stride = head_size;
  p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.head_size = head_size; p.rot_dim = head_size;
  p.cos = cos_sin_cache; p.sin = cos_sin_cache + head_size / 2;
  p.cs_row_stride = head_size; p.positions = positions;
  p.v_src = value; p.v_stride = value_stride; p.k_copy = k_buffer; p.v_copy = v_buffer; p.copy_stride = buffer_row_stride;
  p.slot_mapping = kv_loc; p.num_slots = buffer_rows;
  p.max_pos = max_position; p.err = pipe_error_ptr();
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec_ok = head_size % 16 == 0 && head_size / 16 <= 256 && aligned16(query) && aligned16(key) && aligned16(value) &&
                      aligned16(cos_sin_cache) && aligned16(k_buffer) && aligned16(v_buffer) && (query_stride * 2) % 16 == 0 &&
                      (key_stride * 2) % 16 == 0 && (value_stride * 2) % 16 == 0 && (buffer_row_stride * 2) % 16 == 0;
  int rc = 1;
  if (vec_ok)
    rc = dtype == MCOP_BF16 ? launch_rope_t<__nv_bfloat16, float, false, 2>(p, tokens, 1, true, s)
                            : launch_rope_t<__half, float, false, 2>(p, tokens, 1, true, s);
  if (rc != 1) return rc;
  // few tokens or an odd layout: the rotation, then the copy of the rotated K rows and the V rows (two launches)
  rc = dtype == MCOP_BF16 ? launch_rope_t<__nv_bfloat16, float, false, 0>(p, tokens, 1, vec_ok, s)
                          : launch_rope_t<__half, float, false, 0>(p, tokens, 1, vec_ok, s);
  if (rc) return rc;
  return mcop_reshape_and_cache_flash(key, value, key_stride, value_stride, k_buffer, v_buffer, buffer_row_stride, 0, head_size, kv_loc, tokens,
                                      num_kv_heads, head_size, 1, buffer_rows, 2, stream);
}

extern "C" int mcop_kv_store_i8(const void* packed_qkv, int64_t qkv_stride_token, int64_t qkv_stride_head,
                                const int32_t* q_lens, const int32_t* accum_q_lens, const int32_t* cache_lens,
                                const int32_t* cache_slot_ids, int8_t* k_cache, int8_t* v_cache, int64_t num_slots, int64_t max_len,
                                int64_t k_stride_slot, int64_t k_stride_head, int64_t k_stride_pos,
                                int64_t v_stride_slot, int64_t v_stride_head, int64_t v_stride_pos,
                                const float* k_scale, const float* v_scale, int batch, int64_t tokens, int q_heads,
                                int kv_heads, int head_dim, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(packed_qkv && q_lens && accum_q_lens && cache_lens && cache_slot_ids && k_cache && v_cache && k_scale && v_scale,
               MCOP_ERR_ARGUMENT, "kv_store_i8: null pointer");
  MCOP_REQUIRE(batch > 0 && tokens >= 0 && tokens <= 0x7fffffffLL && q_heads >= 0 && kv_heads > 0 && head_dim > 0 && num_slots > 0 &&
                   max_len > 0, MCOP_ERR_ARGUMENT, "kv_store_i8: bad sizes");
  MCOP_REQUIRE(dtype == MCOP_BF16 || dtype == MCOP_F16, MCOP_ERR_UNSUPPORTED, "kv_store_i8: only f16 and bf16");
  if (tokens == 0) return MCOP_OK;
  KvStoreParams p{packed_qkv, qkv_stride_token, qkv_stride_head, q_lens, accum_q_lens, cache_lens, cache_slot_ids,
                  k_cache, v_cache, k_stride_slot, k_stride_head, k_stride_pos, v_stride_slot, v_stride_head, v_stride_pos,
                  k_scale, v_scale, batch, q_heads, kv_heads, head_dim, num_slots, max_len, pipe_error_ptr()};
  cudaStream_t s = (cudaStream_t)stream;
  const int per_token = 2 * kv_heads * (head_dim >> 4);
  const auto m16 = [](int64_t v) { return v % 16 == 0; };
  const bool vec_ok = head_dim % 16 == 0 && per_token <= 256 && aligned16(packed_qkv) && (qkv_stride_token * 2) % 16 == 0 &&
                      (qkv_stride_head * 2) % 16 == 0 && aligned16(k_cache) && aligned16(v_cache) && aligned16(k_scale) && aligned16(v_scale) &&
                      m16(k_stride_slot) && m16(k_stride_head) && m16(k_stride_pos) && m16(v_stride_slot) && m16(v_stride_head) && m16(v_stride_pos);
  if (vec_ok) {
    // consecutive tokens per thread, measured at 65,536 tokens of 8 + 8 heads: 2 / 4 / 8 -> 93 / 84 / 99 us; with 8 elements per
    // thread and token instead of 16 (consecutive 16-byte loads across a warp, 8-byte stores): 117 us, with 32: 113 us;
    // the token-independent address parts formed once per thread and the sequence's bounds read once per group: 84 -> 74 us
    constexpr int U = 4;
    const int gpc = 256 / per_token;  // token groups per CTA
    const unsigned grid = (unsigned)((tokens + (int64_t)gpc * U - 1) / ((int64_t)gpc * U));
    if (dtype == MCOP_BF16) kv_store_vec<__nv_bfloat16, U><<<grid, gpc * per_token, 0, s>>>(p, tokens, gpc);
    else kv_store_vec<__half, U><<<grid, gpc * per_token, 0, s>>>(p, tokens, gpc);
  } else {
    if (dtype == MCOP_BF16) kv_store_kernel<__nv_bfloat16><<<(unsigned)tokens, 256, 0, s>>>(p);
    else kv_store_kernel<__half><<<(unsigned)tokens, 256, 0, s>>>(p);
  }
  return check_launch("kv_store_i8");
}

extern "C" int mcop_reshape_and_cache_flash(const void* key, const void* value, int64_t key_stride, int64_t value_stride,
                                            void* key_cache, void* value_cache, int64_t block_stride, int64_t page_stride,
                                            int64_t head_stride, const int64_t* slot_mapping, int64_t tokens,
                                            int kv_heads, int head_size, int block_size, int64_t num_blocks, int elem_bytes,
                                            mcop_stream_t stream) {
  MCOP_REQUIRE(key && value && key_cache && value_cache && slot_mapping, MCOP_ERR_ARGUMENT, "reshape_and_cache_flash: null pointer");
  MCOP_REQUIRE(tokens >= 0 && tokens <= 0x7fffffffLL && kv_heads > 0 && head_size > 0 && block_size > 0 && num_blocks >= 0 &&
                   (elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4),
               MCOP_ERR_ARGUMENT, "reshape_and_cache_flash: bad sizes");
  if (tokens == 0) return MCOP_OK;
  CacheCopyParams p{(const char*)key, (const char*)value, key_stride * elem_bytes, value_stride * elem_bytes,
                    (char*)key_cache, (char*)value_cache, block_stride * elem_bytes, page_stride * elem_bytes,
                    head_stride * elem_bytes, slot_mapping, kv_heads, head_size * elem_bytes, block_size,
                    num_blocks * block_size, pipe_error_ptr()};
  const bool v16 = p.head_bytes % 16 == 0 && aligned16(key) && aligned16(value) && aligned16(key_cache) && aligned16(value_cache) &&
                   p.key_stride % 16 == 0 && p.value_stride % 16 == 0 && p.block_stride % 16 == 0 && p.page_stride % 16 == 0 &&
                   p.head_stride % 16 == 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int nvec = kv_heads * (p.head_bytes >> 4);  // 16-byte vectors per token and tensor
  if (v16 && nvec <= 256 && tokens >= 1024) {
    constexpr int U = 4;
    const int tpp = 256 / nvec;  // tokens per pass of the CTA
    const unsigned grid = (unsigned)((tokens + (int64_t)tpp * U - 1) / ((int64_t)tpp * U));
    cache_copy_vec16_multi<U><<<grid, tpp * nvec, 0, s>>>(p, tokens, tpp);
  } else if (v16) cache_copy_kernel<uint4><<<(unsigned)tokens, 256, 0, s>>>(p);
  else if (elem_bytes == 4) cache_copy_kernel<uint32_t><<<(unsigned)tokens, 256, 0, s>>>(p);
  else if (elem_bytes == 2) cache_copy_kernel<uint16_t><<<(unsigned)tokens, 256, 0, s>>>(p);
  else cache_copy_kernel<uint8_t><<<(unsigned)tokens, 256, 0, s>>>(p);
  return check_launch("reshape_and_cache_flash");
}

extern "C" int mcop_reshape_and_cache(const void* key, const void* value, int64_t key_stride, int64_t value_stride,
                                      void* key_cache, void* value_cache, const int64_t* slot_mapping, int64_t tokens,
                                      int kv_heads, int head_size, int block_size, int x, int64_t num_blocks, int elem_bytes,
                                      mcop_stream_t stream) {
  MCOP_REQUIRE(key && value && key_cache && value_cache && slot_mapping, MCOP_ERR_ARGUMENT, "reshape_and_cache: null pointer");
  MCOP_REQUIRE(tokens >= 0 && tokens <= 0x7fffffffLL && kv_heads > 0 && head_size > 0 && block_size > 0 && num_blocks >= 0 && x > 0 &&
                   head_size % x == 0 && (elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4),
               MCOP_ERR_ARGUMENT, "reshape_and_cache: bad sizes (head_size must be a multiple of x)");
  if (tokens == 0) return MCOP_OK;
  CacheSplitParams p{key, value, key_stride, value_stride, key_cache, value_cache, slot_mapping, kv_heads, head_size, block_size, x,
                     num_blocks * block_size, pipe_error_ptr()};
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = (unsigned)tokens;
  // a K group of x elements moves as one 16- or 8-byte vector when it is one and everything is aligned to it
  const int gb = x * elem_bytes;
  const auto al = [&](const void* q, int a) { return (reinterpret_cast<uintptr_t>(q) % a) == 0; };
  const bool g16 = gb == 16 && al(key, 16) && al(key_cache, 16) && (key_stride * elem_bytes) % 16 == 0;
  const bool g8 = gb == 8 && al(key, 8) && al(key_cache, 8) && (key_stride * elem_bytes) % 8 == 0;
  if (elem_bytes == 2) {
    // from a few windows of tokens on, with rows that move as 16-byte vectors and a window that fits shared memory:
    // the tiled kernel (V written run by run instead of element by element)
    const size_t tile_bytes = (size_t)kSplitWindow * kv_heads * head_size * 2;
    if (tokens >= 4 * kSplitWindow && (kv_heads * head_size) % 8 == 0 && al(value, 16) && (value_stride * 2) % 16 == 0 &&
        al(value_cache, 16) && tile_bytes <= 160 * 1024) {
      const unsigned wgrid = (unsigned)((tokens + kSplitWindow - 1) / kSplitWindow);
      auto launch_tile = [&](auto kernel) -> int {
        const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), 200 * 1024);
        MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "reshape_and_cache: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        kernel<<<wgrid, 256, tile_bytes, s>>>(p, tokens);
        return check_launch("reshape_and_cache (tiled)");
      };
      if (g16) return launch_tile(cache_split_tile_kernel<uint4>);
      if (g8) return launch_tile(cache_split_tile_kernel<uint2>);
      return launch_tile(cache_split_tile_kernel<uint16_t>);
    }
    if (g16) cache_split_kernel<uint16_t, uint4><<<grid, 256, 0, s>>>(p);
    else if (g8) cache_split_kernel<uint16_t, uint2><<<grid, 256, 0, s>>>(p);
    else cache_split_kernel<uint16_t, uint16_t><<<grid, 256, 0, s>>>(p);
  } else if (elem_bytes == 4) {
    if (g16) cache_split_kernel<uint32_t, uint4><<<grid, 256, 0, s>>>(p);
    else if (g8) cache_split_kernel<uint32_t, uint2><<<grid, 256, 0, s>>>(p);
    else cache_split_kernel<uint32_t, uint32_t><<<grid, 256, 0, s>>>(p);
  } else {
    if (g16) cache_split_kernel<uint8_t, uint4><<<grid, 256, 0, s>>>(p);
    else if (g8) cache_split_kernel<uint8_t, uint2><<<grid, 256, 0, s>>>(p);
    else cache_split_kernel<uint8_t, uint8_t><<<grid, 256, 0, s>>>(p);
  }
  return check_launch("reshape_and_cache");
}
