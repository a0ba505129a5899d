// Included by rope_kv.cu inside namespace mcop::{anonymous}, after RopeParams, rotate8 and quant8.
//
// Persistent, pipelined NeoX RoPE (+ optional fused KV store: STORE 1 = int8 codes into a paged cache, STORE 2 = the rotated
// K and the V rows copied in the element type to k_copy / v_copy at row slot_mapping[t]) for bf16/f16 activations whose
// heads are contiguous.  A CTA takes chunks of up to 64 consecutive tokens; the positions and slots of the chunk are staged
// in shared memory, then every token's q row, k row, (v row) and cos||sin row arrive in one ring stage by bulk
// asynchronous copies while the CTA rotates, stores and quantises the token before it.
//
// Ring stage layout (bytes): [q: Hq*D*es][k: Hkv*D*es][v: Hkv*D*es if STORE][cos||sin: rot_dim*cs], every part a
// multiple of 16 bytes.

constexpr int kRopeChunk = 64;
constexpr int kRopeMaxKvHeads = 128;  // more KV heads than this use the token-per-CTA kernel

// 80 registers per thread (no spills in any instantiation): four CTAs of six warps then fit the register file of an
// SM, which is split over its four schedulers (24 warps = 6 per scheduler x 32 lanes x 80 registers).
template <typename T, typename CT, bool PER_OP, int STORE>
__global__ void __maxnreg__(80) rope_neox_pipe(RopeParams p, int64_t tokens, int stages, int chunk, int* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int64_t s_pos[kRopeChunk];
  __shared__ int64_t s_slot[kRopeChunk];
  __shared__ float s_kinv[kRopeMaxKvHeads], s_vinv[kRopeMaxKvHeads];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  unsigned char* buf = smem + 128;
  const int D = p.head_size, half = D >> 1, hv = half >> 3;
  const uint32_t q_bytes = (uint32_t)(p.num_heads * D * sizeof(T));
  const uint32_t k_bytes = (uint32_t)(p.num_kv_heads * D * sizeof(T));
  const uint32_t v_bytes = STORE ? k_bytes : 0u;
  const uint32_t cs_bytes = (uint32_t)(p.rot_dim * sizeof(CT));
  const uint32_t stage_bytes = q_bytes + k_bytes + v_bytes + cs_bytes;
  const int j = threadIdx.x % hv;           // slice of the head this thread owns (blockDim % hv == 0)
  const int heads_per_iter = blockDim.x / hv;
  const int nqk = p.num_heads + p.num_kv_heads;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  pdl_wait();  // nothing of global memory is touched before the kernels ahead in the stream have completed
  if (STORE == 1) {
    // reciprocal scales once per CTA: the token loop then reads them from shared memory, not from global memory
    for (int h = threadIdx.x; h < p.num_kv_heads; h += blockDim.x) {
      s_kinv[h] = 1.0f / p.k_scale[h];
      s_vinv[h] = 1.0f / p.v_scale[h];
    }
  }
  __syncthreads();

  uint32_t it = 0, issued = 0;
  RingPos cons, prod;  // ring positions of the consumer (all threads) and of the producer (thread 0)
  bool alive = true;
  // every CTA owns one contiguous share of the tokens (equal to within one token) and walks it in chunks
  const int64_t tok_begin = (tokens * (int64_t)blockIdx.x) / gridDim.x;
  const int64_t tok_end = (tokens * ((int64_t)blockIdx.x + 1)) / gridDim.x;
  for (int64_t t0 = tok_begin; t0 < tok_end && alive; t0 += chunk) {
    const int ntok = (int)min((int64_t)chunk, tok_end - t0);
    if (threadIdx.x < ntok) {
      int64_t pos = token_position(p, t0 + threadIdx.x);  // explicit, or from the bounds of the token's sequence
      if (pos < 0 || pos >= p.max_pos) {  // never becomes an address: the token is skipped (marked by -1) and reported
        report_device_error(p.err, MCOP_DEVERR_POSITION);
        pos = -1;
      }
      s_pos[threadIdx.x] = pos;
      if (STORE) {
        int64_t slot = p.slot_mapping[t0 + threadIdx.x];
        if (slot >= p.num_slots) {
          report_device_error(p.err, MCOP_DEVERR_SLOT);
          slot = -1;
        }
        s_slot[threadIdx.x] = slot;
      }
    }
    __syncthreads();
    int pi = 0;  // producer cursor (thread 0)
    auto issue_next = [&]() {
      if (pi >= ntok) return;
      const int s = prod.s;
      unsigned char* dst = buf + (size_t)s * stage_bytes;
      const int64_t t = t0 + pi;
      mbar_expect_tx(&full[s], stage_bytes);
      bulk_g2s(dst, reinterpret_cast<const T*>(p.q_src) + t * p.q_stride, q_bytes, &full[s]);
      bulk_g2s(dst + q_bytes, reinterpret_cast<const T*>(p.k_src) + t * p.k_stride, k_bytes, &full[s]);
      if (STORE) bulk_g2s(dst + q_bytes + k_bytes, reinterpret_cast<const T*>(p.v_src) + t * p.v_stride, v_bytes, &full[s]);
      // a skipped token still fills its stage (row 0 of the table stands in): the ring stays in step, nothing is used
      const int64_t cs_row = s_pos[pi] < 0 ? 0 : s_pos[pi];
      unsigned char* cs_dst = dst + q_bytes + k_bytes + v_bytes;
      if (p.cs_row_stride == p.rot_dim) {  // cos || sin is one row of one table
        bulk_g2s(cs_dst, reinterpret_cast<const CT*>(p.cos) + cs_row * p.cs_row_stride, cs_bytes, &full[s]);
      } else {                             // two tables of half rows: they land side by side in the stage
        bulk_g2s(cs_dst, reinterpret_cast<const CT*>(p.cos) + cs_row * p.cs_row_stride, cs_bytes / 2, &full[s]);
        bulk_g2s(cs_dst + cs_bytes / 2, reinterpret_cast<const CT*>(p.sin) + cs_row * p.cs_row_stride, cs_bytes / 2, &full[s]);
      }
      ++issued; ++pi;
      prod.advance(stages);
    };
    if (threadIdx.x == 0)
      for (int s = 0; s < stages; ++s) issue_next();
    for (int tl = 0; tl < ntok; ++tl) {
      const int s = cons.s;
      const bool ok = mbar_wait_bounded(&full[s], cons.phase, err, 7);
      if (ok && s_pos[tl] >= 0) {
        const int64_t t = t0 + tl;
        const unsigned char* st = buf + (size_t)s * stage_bytes;
        const T* qs = reinterpret_cast<const T*>(st);
        const T* ks = reinterpret_cast<const T*>(st + q_bytes);
        const CT* cs = reinterpret_cast<const CT*>(st + q_bytes + k_bytes + v_bytes);
        float cc[8], ss[8];
        if (sizeof(CT) == 4) {
          const uint4 a = lds_u4(cs + j * 8), b = lds_u4(cs + j * 8 + 4);
          const uint4 e = lds_u4(cs + half + j * 8), f = lds_u4(cs + half + j * 8 + 4);
          cc[0] = __uint_as_float(a.x); cc[1] = __uint_as_float(a.y); cc[2] = __uint_as_float(a.z); cc[3] = __uint_as_float(a.w);
          cc[4] = __uint_as_float(b.x); cc[5] = __uint_as_float(b.y); cc[6] = __uint_as_float(b.z); cc[7] = __uint_as_float(b.w);
          ss[0] = __uint_as_float(e.x); ss[1] = __uint_as_float(e.y); ss[2] = __uint_as_float(e.z); ss[3] = __uint_as_float(e.w);
          ss[4] = __uint_as_float(f.x); ss[5] = __uint_as_float(f.y); ss[6] = __uint_as_float(f.z); ss[7] = __uint_as_float(f.w);
        } else if (sizeof(T) == 2 && ElemTraits<CT>::code == MCOP_BF16) {
          unpack_bf16x8(lds_u4(cs + j * 8), cc);
          unpack_bf16x8(lds_u4(cs + half + j * 8), ss);
        } else {
          unpack_f16x8(lds_u4(cs + j * 8), cc);
          unpack_f16x8(lds_u4(cs + half + j * 8), ss);
        }
        const int64_t slot = STORE ? s_slot[tl] : -1;
        const CosSin8 cs8 = make_cos_sin(cc, ss);
        for (int h = threadIdx.x / hv; h < nqk; h += heads_per_iter) {
          const bool is_k = h >= p.num_heads;
          const int hh = is_k ? h - p.num_heads : h;
          const T* src = (is_k ? ks : qs) + hh * D;
          T* dst = (is_k ? reinterpret_cast<T*>(p.k_dst) + t * p.k_stride : reinterpret_cast<T*>(p.q_dst) + t * p.q_stride) + hh * D;
          float x[8], y[8], xo[8], yo[8];
          if constexpr (ElemTraits<T>::code == MCOP_BF16 && !PER_OP) {
            // packed path: fewer than half the instructions of the scalar form, same roundings
            uint4 xp, yp;
            rotate_bf16x8_packed(lds_u4(src + j * 8), lds_u4(src + half + j * 8), cs8, xp, yp);
            st_u4(dst + j * 8, xp);
            st_u4(dst + half + j * 8, yp);
            if (STORE == 1 && is_k && slot >= 0) {
              unpack_bf16x8(xp, xo);
              unpack_bf16x8(yp, yo);
            }
            if (STORE == 2 && is_k && slot >= 0) {
              T* kc = reinterpret_cast<T*>(p.k_copy) + slot * p.copy_stride + hh * D;
              st_u4(kc + j * 8, xp);
              st_u4(kc + half + j * 8, yp);
            }
          } else {
            if (ElemTraits<T>::code == MCOP_BF16) {
              unpack_bf16x8(lds_u4(src + j * 8), x);
              unpack_bf16x8(lds_u4(src + half + j * 8), y);
            } else {
              unpack_f16x8(lds_u4(src + j * 8), x);
              unpack_f16x8(lds_u4(src + half + j * 8), y);
            }
            rotate8<T, PER_OP>(x, y, cc, ss, xo, yo);
            Vec8<T>::store(dst + j * 8, xo);
            Vec8<T>::store(dst + half + j * 8, yo);
            if (STORE == 2 && is_k && slot >= 0) {
              T* kc = reinterpret_cast<T*>(p.k_copy) + slot * p.copy_stride + hh * D;
              Vec8<T>::store(kc + j * 8, xo);
              Vec8<T>::store(kc + half + j * 8, yo);
            }
          }
          if (STORE == 1 && is_k && slot >= 0) {
            const float inv = s_kinv[hh];
            int8_t* kc = p.k_cache + (slot * p.num_kv_heads + hh) * (int64_t)D;
            st_cs_u2(kc + j * 8, quant8(xo, inv));
            st_cs_u2(kc + half + j * 8, quant8(yo, inv));
          }
        }
        if constexpr (STORE == 2) if (slot >= 0) {
          // the V row as it came: 16-byte vectors from the stage to the token's row of the buffer
          const unsigned char* vs = st + q_bytes + k_bytes;
          unsigned char* vc = reinterpret_cast<unsigned char*>(reinterpret_cast<T*>(p.v_copy) + slot * p.copy_stride);
          for (uint32_t i = threadIdx.x * 16u; i < v_bytes; i += blockDim.x * 16u) st_u4(vc + i, lds_u4(vs + i));
        }
        if (STORE == 1 && slot >= 0) {
          const T* vs = reinterpret_cast<const T*>(st + q_bytes + k_bytes);
          const int vper = D >> 4;
          const int nitems = p.num_kv_heads * vper;
          for (int i = threadIdx.x; i < nitems; i += blockDim.x) {
            const int hh = i / vper, e = (i % vper) * 16;
            float a[8], b[8];
            if (ElemTraits<T>::code == MCOP_BF16) {
              unpack_bf16x8(lds_u4(vs + hh * D + e), a);
              unpack_bf16x8(lds_u4(vs + hh * D + e + 8), b);
            } else {
              unpack_f16x8(lds_u4(vs + hh * D + e), a);
              unpack_f16x8(lds_u4(vs + hh * D + e + 8), b);
            }
            const float inv = s_vinv[hh];
            const uint2 qa = quant8(a, inv), qb = quant8(b, inv);
            st_cs_u4(p.v_cache + (slot * p.num_kv_heads + hh) * (int64_t)D + e, make_uint4(qa.x, qa.y, qb.x, qb.y));
          }
        }
      }
      // one barrier per token: agrees on success and tells that every thread has left the stage buffer
      if (!__syncthreads_and(ok)) { alive = false; break; }
      ++it;
      cons.advance(stages);
      if (threadIdx.x == 0) {
        proxy_fence_before_reuse();
        issue_next();
      }
    }
    __syncthreads();  // s_pos / s_slot are rewritten by the next chunk
  }
  if (!alive && threadIdx.x == 0) {
    for (uint32_t k = it; k < issued; ++k, cons.advance(stages))
      (void)mbar_wait_bounded(&full[cons.s], cons.phase, err, 8);
  }
}

// Returns MCOP_OK / an error, or 1 when the shape does not fit the pipelined kernel.
template <typename T, typename CT, bool PER_OP, int STORE>
int launch_rope_pipe(const RopeParams& p, int64_t tokens, cudaStream_t stream) {
  const int D = p.head_size, hv = D >> 4;
  if (hv < 1 || 256 % hv != 0 || p.num_kv_heads > kRopeMaxKvHeads) return 1;
  const size_t stage_bytes = (size_t)(p.num_heads + p.num_kv_heads * (STORE ? 2 : 1)) * D * sizeof(T) + (size_t)p.rot_dim * sizeof(CT);
  // block size: the (Hq + Hkv) heads are walked in `iters` rounds of `hpi` heads, chosen so that every round is
  // full (72 heads -> 3 rounds of 24 heads = 192 threads at D = 128) instead of leaving a ragged last round
  const int nqk = p.num_heads + p.num_kv_heads;
  const int hpi_max = 256 / hv;
  const int iters = (nqk + hpi_max - 1) / hpi_max;
  const int hpi = (nqk + iters - 1) / iters;
  int threads = hpi * hv;
  if (threads < 64) threads = 64 / hv * hv;  // chunk staging needs >= 64 threads
  if (threads > 256 || threads % hv != 0) return 1;
  {
    const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&rope_neox_pipe<T, CT, PER_OP, STORE>), 200 * 1024);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "rope: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  // CTAs per SM: try four, then fewer; each gets its share of shared memory for the ring (at least two stages).
  // The runtime is asked how many CTAs really fit: a grid larger than what is resident would run in uneven waves.
  // Measured at 64/8 heads of 128: four CTAs with two stages each 5.69 TB/s, three with three stages 5.52 TB/s.
  int stages = 0, per_sm = 0;
  size_t smem = 0;
  for (int want = 4; want >= 1 && per_sm == 0; --want) {
    int st = (int)(((227 * 1024) / want - 4 * 1024) / stage_bytes);
    if (st < 2) continue;
    if (st > 6) st = 6;
    const size_t sm_bytes = 128 + (size_t)st * stage_bytes;
    int fit = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fit, rope_neox_pipe<T, CT, PER_OP, STORE>, threads, sm_bytes) != cudaSuccess) {
      (void)cudaGetLastError();
      fit = 0;
    }
    if (fit >= want) { stages = st; smem = sm_bytes; per_sm = want; }
  }
  if (per_sm == 0) return 1;
  int64_t grid = (int64_t)sm_count() * per_sm;
  if (grid > (tokens + 7) / 8) grid = (tokens + 7) / 8;
  // (chunks of 32 / 16 / 8 tokens instead of 64: 236-238 us either way at 32,768 tokens of 64/8 heads - the staging of a
  // chunk is one round trip and not what the run waits for)
  const int chunk = kRopeChunk;
  (void)launch_pdl(rope_neox_pipe<T, CT, PER_OP, STORE>, dim3((unsigned)grid), dim3(threads), smem, stream, p, tokens, stages, chunk,
                   pipe_error_ptr());
  return check_launch("rope (pipelined)");
}
