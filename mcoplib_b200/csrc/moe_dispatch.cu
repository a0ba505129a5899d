// Part 3b of the hot path: MoE dispatch (scatter + per-row int8 quantisation) and combine (gather).
//
// Scatter is a deterministic counting sort, not a sort:
//   rank kernel   - one CTA per tile of 512 tokens builds, in shared memory, one bitmap of the tile's
//                   tokens per expert; popcounts give the tile's per-expert histogram and the rank of every
//                   (token, slot) among the tile's rows of that expert.  The last CTA to finish (one atomic
//                   ticket, nobody waits) turns the histograms into per-tile bases, counts and starts.
//   quant kernel  - one CTA per token reads the token row ONCE into registers and emits its k rows at
//                   row = starts[e] + tile_base[tile][e] + rank, i.e. ordered by (expert, token).
// Gather sums the rows of a token in ascending row order in fp32 and rounds once, so the result does not
// depend on scheduling (the reference's bf16 atomics do).
#include "common.cuh"

namespace mcop {
namespace {

constexpr int kTileTokens = 512;
constexpr int kTileWords = kTileTokens / 32;
constexpr int kMaxExperts = 1024;

struct ScatterWs {
  int32_t* ticket;     // 1 int (first 64 ints reserved)
  int32_t* tile_hist;  // [tiles, E] histogram, overwritten by the exclusive per-expert prefix over tiles
  int32_t* rank;       // [T*k] rank of the (token, slot) inside its tile and expert, -1 if dropped
};

__host__ __device__ inline int64_t scatter_tiles(int64_t tokens) { return (tokens + kTileTokens - 1) / kTileTokens; }

// dynamic shared memory: bitmap [E][kTileWords] u32, then prefix [E][kTileWords] u16
__global__ void __launch_bounds__(256) scatter_rank_kernel(const int32_t* __restrict__ ids, ScatterWs ws,
                                                           int32_t* __restrict__ counts, int32_t* __restrict__ starts,
                                                           int64_t tokens, int topk, int E) {
  extern __shared__ uint32_t smem[];
  uint32_t* bitmap = smem;
  uint16_t* prefix = reinterpret_cast<uint16_t*>(smem + (size_t)E * kTileWords);
  __shared__ int is_last;
  const int64_t tile = blockIdx.x;
  const int64_t tok0 = tile * kTileTokens;
  const int ntok = (int)min((int64_t)kTileTokens, tokens - tok0);
  for (int i = threadIdx.x; i < E * kTileWords; i += blockDim.x) bitmap[i] = 0;
  __syncthreads();
  const int32_t* tids = ids + tok0 * topk;
  const int n = ntok * topk;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = tids[i];
    if (e >= 0 && e < E) {
      const int tl = i / topk;
      atomicOr(&bitmap[e * kTileWords + (tl >> 5)], 1u << (tl & 31));
    }
  }
  __syncthreads();
  // one half-warp per expert: exclusive prefix of the 16 word popcounts
  {
    const int hw = threadIdx.x >> 4, l = threadIdx.x & 15, nhw = blockDim.x >> 4;
    for (int e0 = 0; e0 < E; e0 += nhw) {  // trip count is uniform over the warp: the shuffles need every lane
      const int e = e0 + hw;
      const bool valid = e < E;
      const int c = valid ? __popc(bitmap[e * kTileWords + l]) : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o, 16);
        if (l >= o) inc += v;
      }
      if (valid) {
        prefix[e * kTileWords + l] = (uint16_t)(inc - c);
        if (l == 15) ws.tile_hist[tile * E + e] = inc;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = tids[i];
    int r = -1;
    if (e >= 0 && e < E) {
      const int tl = i / topk, wd = tl >> 5;
      r = prefix[e * kTileWords + wd] + __popc(bitmap[e * kTileWords + wd] & ((1u << (tl & 31)) - 1u));
    }
    ws.rank[tok0 * topk + i] = r;
  }
  // ticket: the last CTA to arrive finishes the job; nobody spins
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(ws.ticket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int ntiles = gridDim.x;
  int32_t* cnt_s = reinterpret_cast<int32_t*>(smem);  // reuse: E ints
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarp) {
    int carry = 0;
    for (int t0 = 0; t0 < ntiles; t0 += 32) {
      const int t = t0 + lane;
      const int c = t < ntiles ? __ldcg(&ws.tile_hist[(int64_t)t * E + e]) : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      if (t < ntiles) ws.tile_hist[(int64_t)t * E + e] = carry + inc - c;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) { cnt_s[e] = carry; counts[e] = carry; }
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < E ? cnt_s[e] : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      if (e < E) starts[e] = carry + inc - c;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
  }
}

struct ScatterQuantParams {
  const __nv_bfloat16* hidden; const int32_t* ids; const float* weights; const float* smooth;
  int8_t* rows; float* row_scales; int32_t* row2tok; const int32_t* starts; int32_t* tok2row;
  const int32_t* tile_base; const int32_t* rank;
  int hidden_size, topk, E;
};

__device__ __forceinline__ int scatter_row_of(const ScatterQuantParams& p, int64_t t, int j, int& e, float& w) {
  e = p.ids[t * p.topk + j];
  if (e < 0 || e >= p.E) return -1;
  // weight of the FIRST slot of the token that holds this expert
  int jf = j;
  for (int i = 0; i < j; ++i)
    if (p.ids[t * p.topk + i] == e) { jf = i; break; }
  w = p.weights[t * p.topk + jf];
  const int64_t tile = t / kTileTokens;
  return p.starts[e] + p.tile_base[tile * p.E + e] + p.rank[t * p.topk + j];
}

__device__ __forceinline__ void row_scale_from_amax(float amax, float& scale_out, float& mul) {
  scale_out = (float)((double)amax * 0.0078740157);
  mul = 127.0f * (1.0f / amax);   // amax == 0 -> inf -> 0 * inf = NaN -> code 0
}

template <int THREADS, int NVEC>
__global__ void __launch_bounds__(THREADS) scatter_quant_vec(ScatterQuantParams p) {
  __shared__ float red[33];
  const int64_t t = blockIdx.x;
  const int nv = p.hidden_size >> 3;
  const __nv_bfloat16* x = p.hidden + t * (int64_t)p.hidden_size;
  float xv[NVEC][8];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nv) Vec8<__nv_bfloat16>::load_nc(x + v * 8, xv[i]);
  }
  for (int j = 0; j < p.topk; ++j) {
    int e; float w = 0.f;
    const int row = scatter_row_of(p, t, j, e, w);
    if (threadIdx.x == 0 && p.tok2row) p.tok2row[t * p.topk + j] = row;
    if (row < 0) continue;  // uniform over the CTA
    const float* sm = p.smooth + (int64_t)e * p.hidden_size;
    float vv[NVEC][8];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nv) {
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(sm + v * 8));
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(sm + v * 8) + 1);
        const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          vv[i][q] = xv[i][q] * w * s[q];
          amax = fmaxf(amax, fabsf(vv[i][q]));
        }
      }
    }
    amax = block_reduce<true>(amax, red);
    float scale, mul;
    row_scale_from_amax(amax, scale, mul);
    if (threadIdx.x == 0) { p.row_scales[row] = scale; p.row2tok[row] = (int32_t)t; }
    int8_t* out = p.rows + (int64_t)row * p.hidden_size;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nv) {
        int c[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) c[q] = q_rn_clamp(vv[i][q] * mul, -127, 127);
        st_cs_u2(out + v * 8, pack_i8x8(c));
      }
    }
  }
}

__global__ void __launch_bounds__(256) scatter_quant_any(ScatterQuantParams p) {
  __shared__ float red[33];
  const int64_t t = blockIdx.x;
  const int H = p.hidden_size;
  const __nv_bfloat16* x = p.hidden + t * (int64_t)H;
  for (int j = 0; j < p.topk; ++j) {
    int e; float w = 0.f;
    const int row = scatter_row_of(p, t, j, e, w);
    if (threadIdx.x == 0 && p.tok2row) p.tok2row[t * p.topk + j] = row;
    if (row < 0) continue;
    const float* sm = p.smooth + (int64_t)e * H;
    float amax = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) amax = fmaxf(amax, fabsf(__bfloat162float(x[i]) * w * sm[i]));
    amax = block_reduce<true>(amax, red);
    float scale, mul;
    row_scale_from_amax(amax, scale, mul);
    if (threadIdx.x == 0) { p.row_scales[row] = scale; p.row2tok[row] = (int32_t)t; }
    int8_t* out = p.rows + (int64_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      out[i] = (int8_t)q_rn_clamp(__bfloat162float(x[i]) * w * sm[i] * mul, -127, 127);
  }
}

// ---------------------------------------------------------------------------------------------
// Gather
// ---------------------------------------------------------------------------------------------
// Inversion pre-pass: per token a counter and up to `cap` row ids (unordered; the gather sorts them).
__global__ void gather_invert_kernel(const int32_t* __restrict__ row2tok, int32_t* cnt, int32_t* list, int64_t rows,
                                     int64_t tokens, int cap) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int t = row2tok[r];
  if (t < 0 || t >= tokens) return;
  const int pos = atomicAdd(&cnt[t], 1);
  if (pos < cap) list[(int64_t)t * cap + pos] = (int32_t)r;
}

struct GatherParams {
  const __nv_bfloat16* y; const int32_t* row2tok; __nv_bfloat16* out;
  const int32_t* tok2row; int topk;            // direct inverse (nullable)
  const int32_t* cnt; const int32_t* list; int cap;   // inverse built by the pre-pass
  const int32_t* topk_ids; const float* topk_weights; const int32_t* starts; int experts;  // weighted form
  int64_t rows; int hidden_size; int weighted; int accumulate;
};

constexpr int kMaxList = 64;   // rows of one token handled without the slow scan

// Collect the rows of token t in ascending order into s_rows[0..n) (and their weights into s_w).
// Returns n, or -1 if the token has more rows than the inverse holds (caller falls back to a scan).
__device__ int gather_collect(const GatherParams& p, int64_t t, int32_t* s_rows, float* s_w, int32_t* s_tmp) {
  __shared__ int s_n;
  int n = 0;
  if (p.tok2row) {
    n = p.topk;
    if (threadIdx.x < n) s_tmp[threadIdx.x] = p.tok2row[t * p.topk + threadIdx.x];
  } else {
    n = p.cnt[t];
    if (n > p.cap || n > kMaxList) return -1;
    if (threadIdx.x < n) s_tmp[threadIdx.x] = p.list[t * (int64_t)p.cap + threadIdx.x];
  }
  if (threadIdx.x == 0) s_n = 0;
  __syncthreads();
  if (threadIdx.x < n) {
    const int r = s_tmp[threadIdx.x];
    if (r >= 0 && r < p.rows) {
      int rank = 0;
      for (int i = 0; i < n; ++i) {
        const int o = s_tmp[i];
        if (o >= 0 && o < p.rows && (o < r || (o == r && i < (int)threadIdx.x))) ++rank;
      }
      s_rows[rank] = r;
      atomicAdd(&s_n, 1);
    }
  }
  __syncthreads();
  n = s_n;
  if (p.weighted && threadIdx.x < n) {
    const int r = s_rows[threadIdx.x];
    // expert owning row r: first e with starts[e+1] > r
    int lo = 0, hi = p.experts - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (p.starts[mid + 1] > r) hi = mid; else lo = mid + 1;
    }
    float w = 0.f;
    for (int j = 0; j < p.topk; ++j)
      if (p.topk_ids[t * p.topk + j] == lo) { w = p.topk_weights[t * p.topk + j]; break; }
    s_w[threadIdx.x] = w;
  }
  __syncthreads();
  return n;
}

template <int THREADS, int NVEC>
__global__ void __launch_bounds__(THREADS) gather_vec(GatherParams p) {
  __shared__ int32_t s_rows[kMaxList];
  __shared__ int32_t s_tmp[kMaxList];
  __shared__ float s_w[kMaxList];
  const int64_t t = blockIdx.x;
  const int nv = p.hidden_size >> 3;
  __nv_bfloat16* out = p.out + t * (int64_t)p.hidden_size;
  float acc[NVEC][8];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (p.accumulate && v < nv) {
      Vec8<__nv_bfloat16>::load(out + v * 8, acc[i]);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[i][q] = 0.f;
    }
  }
  const int n = gather_collect(p, t, s_rows, s_w, s_tmp);
  if (n >= 0) {
    for (int r0 = 0; r0 < n; r0 += 4) {
      uint4 raw[4][NVEC];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r0 + u < n) {
          const __nv_bfloat16* src = p.y + (int64_t)s_rows[r0 + u] * p.hidden_size;
#pragma unroll
          for (int i = 0; i < NVEC; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (v < nv) raw[u][i] = ld_nc_u4(src + v * 8);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r0 + u < n) {
          const float w = p.weighted ? s_w[r0 + u] : 1.f;
#pragma unroll
          for (int i = 0; i < NVEC; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (v < nv) {
              float f[8];
              unpack_bf16x8(raw[u][i], f);
#pragma unroll
              for (int q = 0; q < 8; ++q) acc[i][q] = __fadd_rn(acc[i][q], p.weighted ? __fmul_rn(w, f[q]) : f[q]);
            }
          }
        }
      }
    }
  } else {
    // slow path: the token owns more rows than the inverse holds; scan row2tok in ascending chunks
    __shared__ int s_m;
    for (int64_t base = 0; base < p.rows; base += THREADS) {
      if (threadIdx.x == 0) s_m = 0;
      __syncthreads();
      const int64_t r = base + threadIdx.x;
      const bool hit = r < p.rows && p.row2tok[r] == (int32_t)t;
      const unsigned bal = __ballot_sync(0xffffffffu, hit);
      if (bal) {  // ordered compaction is not needed: chunks are <= THREADS rows, handled one by one below
        if ((threadIdx.x & 31) == 0) atomicAdd(&s_m, __popc(bal));
      }
      __syncthreads();
      if (s_m) {
        for (int i = 0; i < THREADS && base + i < p.rows; ++i) {
          if (p.row2tok[base + i] != (int32_t)t) continue;   // uniform: every thread reads the same entry
          const int rr = (int)(base + i);
          float w = 1.f;
          if (p.weighted) {
            int lo = 0, hi = p.experts - 1;
            while (lo < hi) {
              const int mid = (lo + hi) >> 1;
              if (p.starts[mid + 1] > rr) hi = mid; else lo = mid + 1;
            }
            w = 0.f;
            for (int j = 0; j < p.topk; ++j)
              if (p.topk_ids[t * p.topk + j] == lo) { w = p.topk_weights[t * p.topk + j]; break; }
          }
          const __nv_bfloat16* src = p.y + (int64_t)rr * p.hidden_size;
#pragma unroll
          for (int k2 = 0; k2 < NVEC; ++k2) {
            const int v = threadIdx.x + k2 * THREADS;
            if (v < nv) {
              float f[8];
              Vec8<__nv_bfloat16>::load_nc(src + v * 8, f);
#pragma unroll
              for (int q = 0; q < 8; ++q) acc[k2][q] = __fadd_rn(acc[k2][q], p.weighted ? __fmul_rn(w, f[q]) : f[q]);
            }
          }
        }
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nv) st_cs_u4(out + v * 8, pack_bf16x8(acc[i]));
  }
}

// Any hidden size / alignment: one thread per element, rows found by the same inverse (or a scan).
__global__ void __launch_bounds__(256) gather_any(GatherParams p) {
  __shared__ int32_t s_rows[kMaxList];
  __shared__ int32_t s_tmp[kMaxList];
  __shared__ float s_w[kMaxList];
  const int64_t t = blockIdx.x;
  const int H = p.hidden_size;
  __nv_bfloat16* out = p.out + t * (int64_t)H;
  const int n = gather_collect(p, t, s_rows, s_w, s_tmp);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float acc = p.accumulate ? __bfloat162float(out[i]) : 0.f;
    if (n >= 0) {
      for (int u = 0; u < n; ++u) {
        const float f = __bfloat162float(p.y[(int64_t)s_rows[u] * H + i]);
        acc = __fadd_rn(acc, p.weighted ? __fmul_rn(s_w[u], f) : f);
      }
    } else {
      for (int64_t r = 0; r < p.rows; ++r) {
        if (p.row2tok[r] != (int32_t)t) continue;
        float w = 1.f;
        if (p.weighted) {
          int lo = 0, hi = p.experts - 1;
          while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (p.starts[mid + 1] > r) hi = mid; else lo = mid + 1;
          }
          w = 0.f;
          for (int j = 0; j < p.topk; ++j)
            if (p.topk_ids[t * p.topk + j] == lo) { w = p.topk_weights[t * p.topk + j]; break; }
        }
        const float f = __bfloat162float(p.y[r * H + i]);
        acc = __fadd_rn(acc, p.weighted ? __fmul_rn(w, f) : f);
      }
    }
    out[i] = __float2bfloat16_rn(acc);
  }
}

int gather_cap(int64_t tokens, int64_t rows) {
  if (tokens <= 0) return 1;
  int64_t c = (rows + tokens - 1) / tokens;
  if (c < 1) c = 1;
  if (c > 32) c = 32;
  return (int)c;
}

int launch_gather(GatherParams p, int64_t tokens, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (tokens == 0) return MCOP_OK;
  MCOP_REQUIRE(tokens <= 0x7fffffffLL && p.rows <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "moe_gather: too many tokens or rows");
  if (p.tok2row) {
    MCOP_REQUIRE(p.topk >= 1 && p.topk <= kMaxList, MCOP_ERR_ARGUMENT, "moe_gather: topk %d out of range with tok2row", p.topk);
  } else {
    const size_t need = mcop_moe_gather_workspace_bytes(tokens, p.rows);
    MCOP_REQUIRE(workspace && workspace_bytes >= need, MCOP_ERR_WORKSPACE, "moe_gather: workspace of %zu bytes needed, %zu given",
                 need, workspace_bytes);
    MCOP_REQUIRE(aligned16(workspace), MCOP_ERR_ARGUMENT, "moe_gather: workspace must be 16-byte aligned");
    int32_t* cnt = reinterpret_cast<int32_t*>(workspace);
    p.cap = gather_cap(tokens, p.rows);
    p.cnt = cnt;
    p.list = cnt + ((tokens + 63) / 64) * 64;
    cudaError_t e = cudaMemsetAsync(cnt, 0, (size_t)tokens * sizeof(int32_t), stream);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_gather: memset: %s", cudaGetErrorString(e));
    if (p.rows > 0) {
      const int64_t blocks = (p.rows + 255) / 256;
      gather_invert_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p.row2tok, cnt, const_cast<int32_t*>(p.list), p.rows, tokens, p.cap);
      const int rc = check_launch("moe_gather (invert)");
      if (rc) return rc;
    }
  }
  const int nv = p.hidden_size >> 3;
  const bool vec_ok = p.hidden_size % 8 == 0 && aligned16(p.y) && aligned16(p.out) && nv <= 4096;
  const unsigned grid = (unsigned)tokens;
  if (!vec_ok) gather_any<<<grid, 256, 0, stream>>>(p);
  else if (nv <= 256) gather_vec<128, 2><<<grid, 128, 0, stream>>>(p);
  else if (nv <= 1024) gather_vec<256, 4><<<grid, 256, 0, stream>>>(p);
  else if (nv <= 2048) gather_vec<512, 4><<<grid, 512, 0, stream>>>(p);
  else gather_vec<1024, 4><<<grid, 1024, 0, stream>>>(p);
  return check_launch("moe_gather");
}

}  // namespace
}  // namespace mcop

using namespace mcop;

extern "C" size_t mcop_moe_scatter_workspace_bytes(int64_t tokens, int topk, int experts_per_rank) {
  if (tokens < 0 || topk < 0 || experts_per_rank < 0) return 0;
  const int64_t tiles = scatter_tiles(tokens);
  return (size_t)(64 + tiles * experts_per_rank + tokens * topk) * sizeof(int32_t);
}

extern "C" int mcop_moe_scatter_quant_i8(const void* hidden, const int32_t* ids, const float* weights,
                                         const float* smooth, int8_t* rows, float* row_scales, int32_t* row2tok,
                                         int32_t* counts, int32_t* starts, int32_t* tok2row, int64_t tokens,
                                         int64_t hidden_size, int topk, int experts_per_rank, void* workspace,
                                         size_t workspace_bytes, mcop_stream_t stream) {
  MCOP_REQUIRE(hidden && ids && weights && smooth && rows && row_scales && row2tok && counts && starts, MCOP_ERR_ARGUMENT,
               "moe_scatter_quant_i8: null pointer");
  MCOP_REQUIRE(tokens >= 0 && hidden_size > 0 && hidden_size <= 0x7fffffff && topk >= 1 && topk <= 64 && experts_per_rank >= 1,
               MCOP_ERR_ARGUMENT, "moe_scatter_quant_i8: bad sizes");
  MCOP_REQUIRE(experts_per_rank <= kMaxExperts, MCOP_ERR_UNSUPPORTED, "moe_scatter_quant_i8: more than %d experts per rank", kMaxExperts);
  MCOP_REQUIRE(tokens * topk <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "moe_scatter_quant_i8: tokens*topk exceeds int32 row ids");
  const size_t need = mcop_moe_scatter_workspace_bytes(tokens, topk, experts_per_rank);
  MCOP_REQUIRE(workspace && workspace_bytes >= need, MCOP_ERR_WORKSPACE, "moe_scatter_quant_i8: workspace of %zu bytes needed, %zu given",
               need, workspace_bytes);
  MCOP_REQUIRE(aligned16(workspace), MCOP_ERR_ARGUMENT, "moe_scatter_quant_i8: workspace must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const int E = experts_per_rank;
  const int64_t tiles = scatter_tiles(tokens);
  ScatterWs ws;
  ws.ticket = reinterpret_cast<int32_t*>(workspace);
  ws.tile_hist = ws.ticket + 64;
  ws.rank = ws.tile_hist + tiles * E;
  if (tokens == 0) {
    cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int32_t) * E, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(starts, 0, sizeof(int32_t) * E, s);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_scatter_quant_i8: memset: %s", cudaGetErrorString(e));
    return MCOP_OK;
  }
  cudaError_t e = cudaMemsetAsync(ws.ticket, 0, sizeof(int32_t), s);
  MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_scatter_quant_i8: memset: %s", cudaGetErrorString(e));
  const size_t smem = (size_t)E * kTileWords * (sizeof(uint32_t) + sizeof(uint16_t));
  if (smem > 48 * 1024) {
    e = cudaFuncSetAttribute(scatter_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_scatter_quant_i8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  scatter_rank_kernel<<<(unsigned)tiles, 256, smem, s>>>(ids, ws, counts, starts, tokens, topk, E);
  int rc = check_launch("moe_scatter_quant_i8 (rank)");
  if (rc) return rc;
  ScatterQuantParams p{reinterpret_cast<const __nv_bfloat16*>(hidden), ids, weights, smooth, rows, row_scales, row2tok,
                       starts, tok2row, ws.tile_hist, ws.rank, (int)hidden_size, topk, E};
  const int nv = (int)(hidden_size >> 3);
  const bool vec_ok = hidden_size % 8 == 0 && aligned16(hidden) && aligned16(smooth) && (reinterpret_cast<uintptr_t>(rows) & 7u) == 0 && nv <= 4096;
  const unsigned grid = (unsigned)tokens;
  if (!vec_ok) scatter_quant_any<<<grid, 256, 0, s>>>(p);
  else if (nv <= 256) scatter_quant_vec<128, 2><<<grid, 128, 0, s>>>(p);
  else if (nv <= 1024) scatter_quant_vec<256, 4><<<grid, 256, 0, s>>>(p);
  else if (nv <= 2048) scatter_quant_vec<512, 4><<<grid, 512, 0, s>>>(p);
  else scatter_quant_vec<1024, 4><<<grid, 1024, 0, s>>>(p);
  return check_launch("moe_scatter_quant_i8 (quant)");
}

extern "C" size_t mcop_moe_gather_workspace_bytes(int64_t tokens, int64_t rows) {
  if (tokens <= 0 || rows < 0) return 0;
  const int64_t cnt = ((tokens + 63) / 64) * 64;
  return (size_t)(cnt + tokens * gather_cap(tokens, rows)) * sizeof(int32_t);
}

extern "C" int mcop_moe_gather(const void* y, const int32_t* row2tok, void* out, const int32_t* tok2row, int topk,
                               int64_t tokens, int64_t rows, int64_t hidden_size, void* workspace,
                               size_t workspace_bytes, mcop_stream_t stream) {
  MCOP_REQUIRE(y && row2tok && out, MCOP_ERR_ARGUMENT, "moe_gather: null pointer");
  MCOP_REQUIRE(tokens >= 0 && rows >= 0 && hidden_size > 0 && hidden_size <= 0x7fffffff, MCOP_ERR_ARGUMENT, "moe_gather: bad sizes");
  GatherParams p{};
  p.y = reinterpret_cast<const __nv_bfloat16*>(y); p.row2tok = row2tok; p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.tok2row = tok2row; p.topk = topk; p.rows = rows; p.hidden_size = (int)hidden_size; p.weighted = 0; p.accumulate = 1;
  return launch_gather(p, tokens, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int mcop_moe_gather_weighted(const void* y, const int32_t* row2tok, const int32_t* topk_ids,
                                        const float* topk_weights, const int32_t* starts, void* out,
                                        const int32_t* tok2row, int accumulate, int64_t tokens, int64_t rows,
                                        int64_t hidden_size, int topk, int experts, void* workspace,
                                        size_t workspace_bytes, mcop_stream_t stream) {
  MCOP_REQUIRE(y && row2tok && topk_ids && topk_weights && starts && out, MCOP_ERR_ARGUMENT, "moe_gather_weighted: null pointer");
  MCOP_REQUIRE(tokens >= 0 && rows >= 0 && hidden_size > 0 && hidden_size <= 0x7fffffff && topk >= 1 && topk <= kMaxList && experts >= 1,
               MCOP_ERR_ARGUMENT, "moe_gather_weighted: bad sizes");
  GatherParams p{};
  p.y = reinterpret_cast<const __nv_bfloat16*>(y); p.row2tok = row2tok; p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.tok2row = tok2row; p.topk = topk; p.topk_ids = topk_ids; p.topk_weights = topk_weights; p.starts = starts;
  p.experts = experts; p.rows = rows; p.hidden_size = (int)hidden_size; p.weighted = 1; p.accumulate = accumulate;
  return launch_gather(p, tokens, workspace, workspace_bytes, (cudaStream_t)stream);
}
