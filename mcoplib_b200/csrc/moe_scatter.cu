// Part 3b of the hot path: MoE dispatch (scatter + per-row int8 quantisation).
//
// Scatter is a deterministic counting sort, not a sort.  Two launches on the main path, no memset, no inter-CTA wait:
//   bitmap kernel - one CTA per tile of 512 tokens builds, in shared memory, one bitmap of the tile's tokens per
//                   expert and writes the bitmaps and their popcounts (the tile's per-expert histogram) to scratch.
//   quant kernel  - persistent CTAs.  Every CTA first folds the [tiles, experts] histogram into the experts' counts and
//                   starts and into the row offset of every (super-tile, expert) pair, in its own shared memory (the
//                   histogram is a few KB; recomputing it per CTA costs less than a scan kernel and its launch gap, and
//                   needs no ticket that somebody would have to zero).  CTAs then take work items (super-tile, expert,
//                   part) in token-major order, so the k readers of a token row run close together in time and the row
//                   comes from HBM once and from L2 afterwards.  An item enumerates its own tokens from the bitmaps
//                   (rank = popcount prefix), looks up each token's slot and routing weight, and writes row2tok /
//                   tok2row itself.  An item's rows are contiguous in the output and share the expert, so the expert's
//                   smooth-scale slice sits in registers for the whole item while the token rows stream through a ring
//                   of shared-memory stages filled by bulk asynchronous copies.  Rows end up ordered by (expert, token).
// Shapes the quant kernel does not take (row length not a multiple of 8, misaligned buffers, very wide rows, few rows,
// more (super-tile, expert) pairs than its table holds) use the general path: a rank kernel (per-slot ranks; with few
// tiles its last CTA - one atomic ticket, nobody waits - scans the histograms, with many tiles a scan kernel does) and a
// row-per-token quant kernel with the same arithmetic.  moe_align_block_size runs on the rank kernel as well.
#include <atomic>

#include "common.cuh"
#include "tma_pipe.cuh"

namespace mcop {
namespace {

constexpr int kTileTokens = 512;
constexpr int kTileWords = kTileTokens / 32;
constexpr int kMaxExperts = 1024;
constexpr int kBatchRows = 64;   // row indices staged in shared memory at a time by the quant kernel
constexpr int kInKernelScanTiles = 64;  // up to this many tiles the rank kernel's last CTA scans them itself

struct ScatterWs {
  int32_t* ticket;     // [0] ticket of the rank kernel, [1] work counter of the quant kernel (64 ints reserved)
  int32_t* tile_hist;  // [tiles, E] histogram, overwritten by the exclusive per-expert prefix over tiles
  int32_t* rank;       // [T*k] rank of the (token, slot) inside its tile and expert, -1 if dropped
  int32_t separate_scan;  // more than kInKernelScanTiles tiles: scatter_scan_kernel follows the rank kernel
  // Only for moe_align_block_size (all zero / null for the scatter):
  const int32_t* expert_map;  // [E] global -> local expert id, -1 = not on this rank; null = identity
  int32_t block_size;         // > 0: starts are padded to multiples of block_size, expert_ids / total are written
  int32_t* expert_ids;        // [max_blocks] expert of every block of block_size sorted positions
  int64_t max_blocks;
  int32_t* total;             // [1] number of sorted positions after padding
  int32_t* prefill;           // [prefill_n] filled with prefill_value by the rank kernel (the "no token" mark)
  int64_t prefill_n;
  int32_t prefill_value;
};

// expert of one routing entry after the optional map; -1 = dropped (out of range, or mapped to -1)
__device__ __forceinline__ int mapped_expert(int e, int E, const int32_t* __restrict__ map) {
  if (e < 0 || e >= E) return -1;
  if (map) {
    e = map[e];
    if (e < 0 || e >= E) return -1;
  }
  return e;
}

__host__ __device__ inline int64_t scatter_tiles(int64_t tokens) { return (tokens + kTileTokens - 1) / kTileTokens; }

// Last step of the counting, run by one whole CTA: cnt_s[0, E) (shared memory, room for 3 E + 1 ints) holds the
// experts' row counts; writes starts[] (exclusive prefix; of the counts padded to block_size in the align form) and,
// in the align form, the expert of every block and the padded total.
__device__ __forceinline__ void finish_experts(int32_t* cnt_s, const ScatterWs& ws, int32_t* __restrict__ starts, int E) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  const int bs = ws.block_size;
  int32_t* pst_s = cnt_s + E;      // padded start and padded count of every expert (align form only)
  int32_t* pcn_s = cnt_s + 2 * E;
  if (warp == 0) {
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      int c = e < E ? cnt_s[e] : 0;
      if (bs > 0) c = (c + bs - 1) / bs * bs;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      if (e < E) {
        starts[e] = carry + inc - c;
        if (bs > 0) { pst_s[e] = carry + inc - c; pcn_s[e] = c; }
      }
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (bs > 0 && lane == 0) { *ws.total = carry; cnt_s[3 * E] = carry; }
  }
  if (bs > 0) {  // uniform over the CTA
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      for (int i = pst_s[e]; i < pst_s[e] + pcn_s[e]; i += bs)
        if (i / bs < ws.max_blocks) ws.expert_ids[i / bs] = e;
    // blocks past the padded total belong to no expert: 0, as the reference fills them
    for (int64_t i = cnt_s[3 * E] / bs + threadIdx.x; i < ws.max_blocks; i += blockDim.x) ws.expert_ids[i] = 0;
  }
}

// dynamic shared memory: bitmap [E][kTileWords] u32, then prefix [E][kTileWords] u16 (16 E words: the 3 E + 1 ints
// of finish_experts fit when the area is reused)
__global__ void __launch_bounds__(256) scatter_rank_kernel(const int32_t* __restrict__ ids, ScatterWs ws,
                                                           int32_t* __restrict__ counts, int32_t* __restrict__ starts,
                                                           int64_t tokens, int topk, int E) {
  extern __shared__ uint32_t smem_u32[];
  uint32_t* bitmap = smem_u32;
  uint16_t* prefix = reinterpret_cast<uint16_t*>(smem_u32 + (size_t)E * kTileWords);
  __shared__ int is_last;
  const int64_t tile = blockIdx.x;
  const int64_t tok0 = tile * kTileTokens;
  const int ntok = (int)min((int64_t)kTileTokens, tokens - tok0);
  for (int i = threadIdx.x; i < E * kTileWords; i += blockDim.x) bitmap[i] = 0;
  if (ws.prefill) {
    const int64_t per = (ws.prefill_n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = per * blockIdx.x, hi = min(lo + per, ws.prefill_n);
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) ws.prefill[i] = ws.prefill_value;
  }
  __syncthreads();
  const int32_t* tids = ids + tok0 * topk;
  const int n = ntok * topk;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = mapped_expert(tids[i], E, ws.expert_map);
    if (e >= 0) {
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
    const int e = mapped_expert(tids[i], E, ws.expert_map);
    int r = -1;
    if (e >= 0) {
      const int tl = i / topk, wd = tl >> 5;
      r = prefix[e * kTileWords + wd] + __popc(bitmap[e * kTileWords + wd] & ((1u << (tl & 31)) - 1u));
    }
    ws.rank[tok0 * topk + i] = r;
  }
  if (ws.separate_scan) return;  // many tiles: scatter_scan_kernel turns the histograms into bases (one CTA per expert)
  // few tiles - ticket: the last CTA to arrive finishes the job; nobody spins
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(ws.ticket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int ntiles = gridDim.x;
  int32_t* cnt_s = reinterpret_cast<int32_t*>(smem_u32);  // reuse: E ints
  // one thread per expert walks the tiles; the loads are coalesced over experts and independent of each other, so
  // they overlap instead of paying one memory latency per expert
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
#pragma unroll 8
    for (int t = 0; t < ntiles; ++t) {
      const int c = __ldcg(&ws.tile_hist[(int64_t)t * E + e]);
      ws.tile_hist[(int64_t)t * E + e] = run;
      run += c;
    }
    cnt_s[e] = run;
    counts[e] = run;
  }
  finish_experts(cnt_s, ws, starts, E);
}

// Second step when there are many tiles: CTA e turns column e of the [tiles, E] histogram into exclusive prefixes
// over the tiles (256 tiles per round, block scan) and writes counts[e]; the last CTA to finish (ticket, nobody
// waits) derives the experts' starts.
__global__ void __launch_bounds__(256) scatter_scan_kernel(ScatterWs ws, int32_t* __restrict__ counts,
                                                           int32_t* __restrict__ starts, int ntiles, int E) {
  __shared__ int32_t wsum[8];
  __shared__ int is_last;
  __shared__ int32_t cnt_s[3 * kMaxExperts + 1];
  const int e = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int carry = 0;
  for (int t0 = 0; t0 < ntiles; t0 += 256) {
    const int t = t0 + threadIdx.x;
    const int c = t < ntiles ? __ldcg(&ws.tile_hist[(int64_t)t * E + e]) : 0;
    int inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += v;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    int base = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int v = wsum[w];
      if (w < warp) base += v;
      tot += v;
    }
    if (t < ntiles) ws.tile_hist[(int64_t)t * E + e] = carry + base + inc - c;
    carry += tot;
    __syncthreads();  // wsum is rewritten by the next round
  }
  if (threadIdx.x == 0) counts[e] = carry;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(ws.ticket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < E; i += blockDim.x) cnt_s[i] = __ldcg(&counts[i]);
  finish_experts(cnt_s, ws, starts, E);
}

// moe_align_block_size, second step: one thread per routing entry writes its flat index to its sorted position.
__global__ void __launch_bounds__(256) align_fill_kernel(const int32_t* __restrict__ ids, ScatterWs ws,
                                                         const int32_t* __restrict__ starts, int32_t* __restrict__ sorted,
                                                         int64_t numel, int E, int64_t cap) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= numel) return;
  const int r = ws.rank[i];
  if (r < 0) return;
  const int e = mapped_expert(ids[i], E, ws.expert_map);
  const int64_t pos = (int64_t)starts[e] + ws.tile_hist[(i / kTileTokens) * E + e] + r;
  if (pos < cap) sorted[pos] = (int32_t)i;
}

struct ScatterQuantParams {
  const __nv_bfloat16* hidden; const int32_t* ids; const float* weights; const float* smooth;
  int8_t* rows; float* row_scales; int32_t* row2tok; int32_t* starts; int32_t* counts; int32_t* tok2row;
  const int32_t* tile_base; const int32_t* rank;   // general path: per-tile bases and per-slot ranks of the rank kernel
  const int32_t* hist; const uint32_t* bitmaps;     // main path: [tiles, E] histogram and [tiles, E, 16] token bitmaps
  int32_t* work_counter;
  int64_t tokens; int hidden_size, topk, E;
  int supertile, parts;   // quant kernel work items: (super-tile of `supertile` tiles, expert, part of `parts`)
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

// ---------------------------------------------------------------------------------------------
// Main path, first launch: per tile, one bitmap of the tile's tokens per expert and its popcount.
// Dynamic shared memory: bitmap [E][kTileWords] u32.  Also resets the work counter of the quant kernel that follows
// in stream order (so nobody has to zero the scratch) and marks the dropped (token, slot) entries in tok2row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) scatter_bitmap_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ hist,
                                                             uint32_t* __restrict__ bitmaps, int32_t* __restrict__ work_counter,
                                                             int32_t* __restrict__ tok2row, int64_t tokens, int topk, int E) {
  extern __shared__ uint32_t smem_u32[];
  uint32_t* bitmap = smem_u32;
  const int64_t tile = blockIdx.x;
  const int64_t tok0 = tile * kTileTokens;
  const int ntok = (int)min((int64_t)kTileTokens, tokens - tok0);
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < E * kTileWords; i += blockDim.x) bitmap[i] = 0;
  pdl_wait();  // nothing of global memory is touched before the kernels ahead in the stream have completed
  if (blockIdx.x == 0 && threadIdx.x == 0) *work_counter = 0;
  __syncthreads();
  const int32_t* tids = ids + tok0 * topk;
  const int n = ntok * topk;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = tids[i];
    if (e >= 0 && e < E) {
      const int tl = i / topk;
      atomicOr(&bitmap[e * kTileWords + (tl >> 5)], 1u << (tl & 31));
    } else if (tok2row) {
      tok2row[tok0 * topk + i] = -1;
    }
  }
  __syncthreads();
  // one half-warp per expert: the 16 words go out as one 64-byte line, their popcounts are summed by shuffles
  const int hw = threadIdx.x >> 4, l = threadIdx.x & 15, nhw = blockDim.x >> 4;
  for (int e0 = 0; e0 < E; e0 += nhw) {  // trip count is uniform over the warp: the shuffles need every lane
    const int e = e0 + hw;
    const bool valid = e < E;
    const uint32_t wv = valid ? bitmap[e * kTileWords + l] : 0u;
    int c = __popc(wv);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o, 16);
    if (valid) {
      bitmaps[(tile * E + e) * kTileWords + l] = wv;
      if (l == 0) hist[tile * E + e] = c;
    }
  }
}

constexpr int kTableMax = 2048;  // (super-tile, expert) pairs whose row offsets a quant CTA keeps in shared memory

__device__ __forceinline__ uint4 lds_u4_at(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
  return r;
}

// Prologue of the quant kernel (every CTA, identical results): folds the [tiles, E] histogram into the experts' counts
// and starts and the row offset of every (super-tile, expert) pair, all in the CTA's shared memory:
// table = starts [E], counts [E], offsets [nsuper, E].  CTA 0 also writes the counts and starts to the caller.
// Kept out of line: its registers are not wanted in the row loop.
__device__ __noinline__ void scatter_fold_histogram(const ScatterQuantParams& p, int32_t* table, int ntiles, int nsuper) {
  const int E = p.E, nthreads = blockDim.x, nwarp = blockDim.x >> 5;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t* s_starts = table;
  int32_t* s_cnt = s_starts + E;
  int32_t* s_base = s_cnt + E;
  const int nent = nsuper * E;
  for (int i = threadIdx.x; i < nent; i += nthreads) {
    const int g = i / E, e = i - g * E;
    const int tl = g * p.supertile, th = min(tl + p.supertile, ntiles);
    int c = 0;
    for (int t = tl; t < th; ++t) c += __ldg(p.hist + (int64_t)t * E + e);
    s_base[i] = c;
  }
  __syncthreads();
  if (E <= 32) {
    // few experts, many super-tiles: one warp per expert column, shuffle scans of 32 super-tiles at a time
    for (int e = warp; e < E; e += nwarp) {
      int carry = 0;
      for (int g0 = 0; g0 < nsuper; g0 += 32) {
        const int g = g0 + lane;
        const int c = g < nsuper ? s_base[g * E + e] : 0;
        int inc = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += v;
        }
        if (g < nsuper) s_base[g * E + e] = carry + inc - c;
        carry += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) s_cnt[e] = carry;
    }
  } else {
    for (int e = threadIdx.x; e < E; e += nthreads) {
      int run = 0;
      for (int g = 0; g < nsuper; ++g) {
        const int c = s_base[g * E + e];
        s_base[g * E + e] = run;
        run += c;
      }
      s_cnt[e] = run;
    }
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < E ? s_cnt[e] : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      if (e < E) s_starts[e] = carry + inc - c;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e < E; e += nthreads) { p.counts[e] = s_cnt[e]; p.starts[e] = s_starts[e]; }
}

// One batch of an item, first half (whole CTA): the tokens holding ranks [lo, lo + nb) of expert e inside tiles
// [tile_lo, tile_hi), in ascending order, go to s_tok.  Ends with a CTA barrier.  One round trip to memory: the bitmaps
// of the (few) tiles are fetched together with their counts.
// Both halves are inlined: as calls they cost the CTA a spill of the live smooth slice to the stack and a reload from
// L2 afterwards (the L1 that is left beside the ring does not keep the stack) - two more round trips per item.
__device__ __forceinline__ void scatter_list_tokens(const ScatterQuantParams& p, int e, int tile_lo, int tile_hi, int lo, int nb, int32_t* s_tok) {
  const int E = p.E;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp == 0) {
    const int hi = lo + nb;
    if (tile_hi - tile_lo <= 2) {
      // one or two tiles: lanes 0-15 take the words of the first tile, lanes 16-31 those of the second
      const int half = lane >> 4, wi = lane & 15;
      const int tt = tile_lo + half;
      const bool have = tt < tile_hi;
      uint32_t wv = have ? __ldg(p.bitmaps + ((int64_t)tt * E + e) * kTileWords + wi) : 0u;
      const int pc = __popc(wv);
      int winc = pc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += v;
      }
      int r = winc - pc;  // rank of the word's first set bit (tiles in order, words in order)
      while (wv) {
        const int bit = __ffs(wv) - 1;
        wv &= wv - 1;
        if (r >= lo && r < hi) s_tok[r - lo] = tt * kTileTokens + wi * 32 + bit;
        ++r;
      }
    } else {
      int run = 0;  // rows of the (super-tile, expert) pair in the tiles before the current group of 32
      for (int c0 = tile_lo; c0 < tile_hi && run < hi; c0 += 32) {
        const int t = c0 + lane;
        const int c = t < tile_hi ? __ldg(p.hist + (int64_t)t * E + e) : 0;
        int inc = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += v;
        }
        const int first = run + inc - c;  // rank of the tile's first row
        unsigned need = __ballot_sync(0xffffffffu, c > 0 && first < hi && first + c > lo);
        while (need) {  // uniform over the warp
          const int b = __ffs(need) - 1;
          need &= need - 1;
          const int tt = c0 + b;
          const int base = __shfl_sync(0xffffffffu, first, b);
          uint32_t wv = lane < kTileWords ? __ldg(p.bitmaps + ((int64_t)tt * E + e) * kTileWords + lane) : 0u;
          const int pc = __popc(wv);
          int winc = pc;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += v;
          }
          int r = base + winc - pc;  // rank of the word's first set bit
          while (wv) {
            const int bit = __ffs(wv) - 1;
            wv &= wv - 1;
            if (r >= lo && r < hi) s_tok[r - lo] = tt * kTileTokens + lane * 32 + bit;
            ++r;
          }
        }
        run += __shfl_sync(0xffffffffu, inc, 31);
      }
    }
  }
  __syncthreads();
}

// Second half: the routing weights of the batch's tokens go to s_wt; row2tok / tok2row of the rows b0 .. b0 + nb - 1 are
// written.  Ends with a CTA barrier.  One round trip: the weights of all slots are fetched together with the ids.
__device__ __forceinline__ void scatter_stage_weights(const ScatterQuantParams& p, int e, int nb, int b0, const int32_t* s_tok, float* s_wt) {
  // slot and routing weight of every token of the batch; the row's entries of row2tok / tok2row
  if (threadIdx.x < nb) {
    const int t = s_tok[threadIdx.x];
    const int row = b0 + threadIdx.x;
    const int32_t* tid = p.ids + (int64_t)t * p.topk;
    const float* tw = p.weights + (int64_t)t * p.topk;
    float w = 0.f;
    if (p.topk <= 8) {
      // ids and weights of all slots in flight at once, the choice afterwards
      int idv[8]; float wv8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        idv[j] = j < p.topk ? tid[j] : -1;
        wv8[j] = j < p.topk ? tw[j] : 0.f;
      }
      bool found = false;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (idv[j] == e) {
          if (!found) { w = wv8[j]; found = true; }  // the weight is that of the FIRST slot of the token that holds this expert
          if (p.tok2row) p.tok2row[(int64_t)t * p.topk + j] = row;
        }
      }
    } else {
      int jf = -1;
      for (int j = 0; j < p.topk; ++j) {
        if (tid[j] == e) {
          if (jf < 0) jf = j;
          if (p.tok2row) p.tok2row[(int64_t)t * p.topk + j] = row;
        }
      }
      w = tw[jf < 0 ? 0 : jf];
    }
    s_wt[threadIdx.x] = w;
    p.row2tok[row] = t;
  }
  __syncthreads();
}

// Main path, second launch: persistent pipelined quant kernel.
// What bounds it at 262,144 tokens x top-2 is not the SM: with the multiply and the two rounding adds of pass 2 taken out
// (a fifth of the instructions) it takes the same 1325-1335 us, and a form that keeps the row's products in tensor
// memory between the passes (tcgen05.alloc of 64 columns per CTA, tcgen05.st / ld of 8 columns, 128 registers, four
// CTAs per SM, bit-identical) takes 1395 us against 1325 (199 against 185 us at 32,768 tokens; only below 8192 tokens
// is it ahead, 39 against 44 us at 4096).  Every token row is read k times, once from DRAM and k - 1 times from L2: at
// top-2 the SMs take in 5.6 TB/s and put out 2.8 TB/s, 8.4 TB/s through the L2, where the kernels that run at 0.98 of
// the copy bandwidth move 6.4-6.5 TB/s; the bytes the roofline counts (a token row once) are 5.7 TB/s of that.
// Dynamic shared memory: 128 bytes of mbarriers; the table (starts [E], counts [E], row offset of every
// (super-tile, expert) pair [nsuper, E]) rounded up to 128 bytes; then `stages` row buffers.
template <int THREADS, int NVEC, bool FULL, int CTAS>  // FULL: the row is exactly THREADS * NVEC vectors of 8, no lane is ever idle
__global__ void __launch_bounds__(THREADS, CTAS) scatter_quant_pipe(ScatterQuantParams p, int stages, int table_bytes, int* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int NWARP = THREADS / 32, RS = (NWARP + 7) / 8 * 8;  // warps, and the slots of one reduction
  __shared__ float red[2][RS];
  __shared__ int32_t s_tok[kBatchRows];
  __shared__ float s_wt[kBatchRows];
  __shared__ int s_item;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  int32_t* s_starts = reinterpret_cast<int32_t*>(smem + 128);
  const int E = p.E;
  int32_t* s_cnt = s_starts + E;
  int32_t* s_base = s_cnt + E;
  unsigned char* buf = smem + 128 + table_bytes;
  const int H = p.hidden_size, nv = H >> 3;
  const uint32_t row_bytes = (uint32_t)H * 2u;
  const int ntiles = (int)scatter_tiles(p.tokens);
  const int nsuper = (ntiles + p.supertile - 1) / p.supertile;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  pdl_wait();  // nothing of global memory is touched before the kernels ahead in the stream have completed
  scatter_fold_histogram(p, s_starts, ntiles, nsuper);

  const uint32_t buf_s = smem_addr(buf) + threadIdx.x * 16u;  // this thread's first vector of stage 0 (shared address)
  uint32_t it = 0, issued = 0, flip = 0;
  RingPos cons, prod;  // ring positions of the consumer (all threads) and of the producer (thread 0)
  bool alive = true;
  const int nitems = nsuper * E * p.parts;
  while (alive) {
    // work items (super-tile, expert, part) from an atomic counter, in token-major order: the CTAs move through the
    // tokens together, so the k readers of a token row run close together in time
    // (asking the counter for the next item while this one runs, so that the atomic's round trip hides behind the rows,
    // measured the same: 1357 / 201 us against 1349-1354 / 199-203 us at 262,144 / 32,768 tokens.
    // Preparing the whole next item while the last rows of this one are quantised - the counter asked a dozen rows before
    // the end, bitmap words and ids / weights brought by asynchronous copies into shared memory, tokens listed, weights
    // chosen, each step between two rows, and the producer running on into the next item's rows - cut the time from an
    // item's start to its first row from 11,000 to 3,600 cycles and still lost: 204 against 185 us at 32,768 tokens,
    // 1470-1600 against 1330-1450 us at 262,144.  With the steps compiled in but switched off it was 201 us: the state
    // they keep alive costs the row loop its registers, and the two other CTAs of the SM were already covering for a
    // CTA that sits in its set-up.)
    if (threadIdx.x == 0) s_item = atomicAdd(p.work_counter, 1);
    __syncthreads();
    const int item = s_item;
    __syncthreads();  // s_item may be rewritten only after everybody has read it
    if (item >= nitems) break;
    // 32-bit arithmetic throughout (64-bit divisions are long instruction sequences, and the CTA waits for them): the host
    // keeps the item count below 2^30, a (super-tile, expert) pair holds at most 64 * 512 rows and is cut into at most 64 parts
    const int part = item % p.parts, pe = item / p.parts;
    const int e = pe % E;
    const int sup = pe / E;
    const int tile_lo = sup * p.supertile;
    const int tile_hi = min(tile_lo + p.supertile, ntiles);
    const int off_lo = s_base[sup * E + e];
    const int nall = (sup + 1 < nsuper ? s_base[(sup + 1) * E + e] : s_cnt[e]) - off_lo;
    const int rb_all = s_starts[e] + off_lo;
    const int lo_part = nall * part / p.parts;
    const int hi_part = nall * (part + 1) / p.parts;
    if (hi_part <= lo_part) continue;  // uniform over the CTA
    // the expert's smooth-scale slice stays in registers for the whole item
    // (kept as pairs: the arithmetic below uses the packed fp32x2 multiply of sm_100)
    float2 sm[NVEC][4];
    {
      const float* smp = p.smooth + (int64_t)e * H;
#pragma unroll
      for (int k = 0; k < NVEC; ++k) {
        const int v = threadIdx.x + k * THREADS;
        if (FULL || v < nv) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(smp + v * 8));
          const float4 b = __ldg(reinterpret_cast<const float4*>(smp + v * 8) + 1);
          sm[k][0] = make_float2(a.x, a.y); sm[k][1] = make_float2(a.z, a.w);
          sm[k][2] = make_float2(b.x, b.y); sm[k][3] = make_float2(b.z, b.w);
        }
      }
    }
    for (int lo = lo_part; lo < hi_part && alive; lo += kBatchRows) {
      const int nb = min(kBatchRows, hi_part - lo);
      const int b0 = rb_all + lo;  // output row of the batch's first token
      scatter_list_tokens(p, e, tile_lo, tile_hi, lo, nb, s_tok);
      int pi = 0;  // producer cursor inside the batch (thread 0)
      auto issue_next = [&]() {
        if (pi >= nb) return;
        const int s = prod.s;
        mbar_expect_tx(&full[s], row_bytes);
        bulk_g2s(buf + (size_t)s * row_bytes, p.hidden + (int64_t)s_tok[pi] * H, row_bytes, &full[s]);
        ++issued; ++pi;
        prod.advance(stages);
      };
      // the first rows are on their way while the ids and weights of the batch are fetched
      if (threadIdx.x == 0)
        for (int s = 0; s < stages; ++s) issue_next();
      scatter_stage_weights(p, e, nb, b0, s_tok, s_wt);
      for (int i = 0; i < nb; ++i) {
        const int st = cons.s;
        const bool ok = mbar_wait_bounded(&full[st], cons.phase, err, 5);
        float2 vv[NVEC][4];
        float amax = 0.f;
        if (ok) {
          const uint32_t src = buf_s + (uint32_t)st * row_bytes;
          const float w = s_wt[i];
          const float2 w2 = make_float2(w, w);
#pragma unroll
          for (int k = 0; k < NVEC; ++k) {
            if (FULL || threadIdx.x + k * THREADS < nv) {
              const uint4 raw = lds_u4_at(src + (uint32_t)(k * THREADS * 16));
              const uint32_t wd[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 x2 = make_float2(__uint_as_float(wd[q] << 16), __uint_as_float(wd[q] & 0xffff0000u));
                vv[k][q] = mul2_rn(mul2_rn(x2, w2), sm[k][q]);  // (x * w) * smooth, each product rounded
                // one running maximum for the whole row: a chain per pass measured no faster
                amax = max3_abs(amax, vv[k][q].x, vv[k][q].y);
              }
            }
          }
        }
        amax = warp_max_nonneg(amax);
        float* rd = red[flip & 1u];
        if (lane == 0) rd[warp] = amax;
        // the single barrier of the row: agrees on success, publishes the warp maxima and tells that every thread
        // has left the stage buffer (the two `red` halves alternate, so no second barrier is needed)
        if (!__syncthreads_and(ok)) { alive = false; break; }
        ++it; ++flip;
        cons.advance(stages);
        if (threadIdx.x == 0) {
          proxy_fence_before_reuse();
          issue_next();
        }
        // max over the NWARP warp maxima: the first NWARP lanes read one each, one warp reduction
        const float m = warp_max_nonneg(lane < NWARP ? rd[lane] : 0.f);
        // all-zero row: codes 0 (keeps NaN out of the bit-level conversion below)
        const float mul = m > 0.f ? 127.0f * (1.0f / m) : 0.f;
        const float2 mul2 = make_float2(mul, mul);
        const int row = b0 + i;
        if (threadIdx.x == 0) p.row_scales[row] = (float)((double)m * 0.0078740157);
        int8_t* out = p.rows + (int64_t)row * H + threadIdx.x * 8;
#pragma unroll
        for (int k = 0; k < NVEC; ++k) {
          if (FULL || threadIdx.x + k * THREADS < nv) {
            // |v * mul| <= 127 * (1 + 2^-22): rounds into [-127, 127], no clamp needed
            uint32_t c[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              // packed product, scalar rounding adds.  Measured: a packed add here gets contracted with the packed product
              // into one fused multiply-add by the assembler (4 % faster, but the codes differ: one rounding instead of
              // two); a packed fma(pr, 1, magic), which cannot be contracted, is exact and no faster than the scalar adds.
              // The row's scale written by another warp than the one that issues the copies: no change either.
              const float2 pr = mul2_rn(vv[k][q], mul2);
              c[2 * q] = rn_low_byte(pr.x);
              c[2 * q + 1] = rn_low_byte(pr.y);
            }
            st_cs_u2(out + k * THREADS * 8, make_uint2(pack4_low_bytes(c[0], c[1], c[2], c[3]), pack4_low_bytes(c[4], c[5], c[6], c[7])));
          }
        }
      }
      __syncthreads();  // s_tok / s_wt are rewritten by the next batch
    }
  }
  if (!alive && threadIdx.x == 0) {
    for (uint32_t k = it; k < issued; ++k, cons.advance(stages))
      (void)mbar_wait_bounded(&full[cons.s], cons.phase, err, 6);
  }
}

// Row-per-token kernels (any shape).  They compute the row index themselves (no fill pass needed).
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

// Returns MCOP_OK / an error, or 1 when the problem does not fit the main path (more (super-tile, expert) pairs than the
// table holds, or no room for the ring).
template <int THREADS, int NVEC, int CTAS>
int launch_quant_pipe(ScatterQuantParams p, cudaStream_t stream) {
  const size_t row_bytes = (size_t)p.hidden_size * 2;
  const int64_t ntiles = scatter_tiles(p.tokens);
  // work items: ~40 rows each amortise the per-item set-up; with few rows in total they shrink (down to 16) so that
  // every CTA still gets half a dozen items from the counter and the tail of the last wave stays short
  const double total_rows = (double)p.tokens * p.topk;
  // (measured at 8192 tokens x top-8 of 256: items of 16 rows +1 %, of 8 rows -4 % against this rule; at 32,768 tokens x
  // top-2 of 8 items of 12 / 16 / 20 / 24 / 32 / 40 / 56 rows: 213 / 209 / 202 / 199 / 197 / 200 / 220 us - flat around the rule's 25;
  // half-size items for the last quarter / half / all of the super-tiles: 200 / 205 / 214 us there, 1370 / 1449 / 1552 us
  // against 1347 us at 262,144 tokens - the spread of the CTAs' finishing times is not what the short runs lose;
  // again after the per-item set-up had lost two round trips: 10 / 13 / 16 / 20 / 32 rows at 32,768 tokens 200 / 191 / 189 /
  // 187 / 185 us against 186 us for the rule, 20 / 26 / 32 / 64 rows at 262,144 tokens 1358 / 1362 / 1375 / 1348 against 1317 us)
  double target = total_rows / ((double)sm_count() * CTAS * 6.0);
  target = target < 16.0 ? 16.0 : (target > 40.0 ? 40.0 : target);
  const double rows_per_tile_expert = (double)kTileTokens * p.topk / p.E;
  int64_t supertile = (int64_t)((target + rows_per_tile_expert - 1e-9) / rows_per_tile_expert);
  if (supertile < 1) supertile = 1;
  // the (super-tile, expert) table of a CTA holds kTableMax pairs: coarser super-tiles (cut into more parts) when needed
  const int64_t max_super = kTableMax / p.E;
  if (max_super < 1) return 1;
  const int64_t need_supertile = (ntiles + max_super - 1) / max_super;
  if (supertile < need_supertile) supertile = need_supertile;
  if (supertile > 64) return 1;
  int parts = (int)(supertile * rows_per_tile_expert / target);
  if (parts < 1) parts = 1;
  if (parts > 64) parts = 64;
  p.supertile = (int)supertile;
  p.parts = parts;
  const int64_t nsuper = (ntiles + supertile - 1) / supertile;
  const int64_t nitems = nsuper * p.E * parts;
  if (nitems >= (int64_t)1 << 30) return 1;  // the kernel numbers its items with 32 bits
  const int table_bytes = (int)(((2 * (int64_t)p.E + nsuper * p.E) * sizeof(int32_t) + 127) / 128 * 128);
  // each of the CTAS resident CTAs gets its share of the shared memory: barriers, table, ring of row buffers
  const int64_t budget = (227 * 1024) / CTAS - 2 * 1024 - 128 - table_bytes;
  int stages = (int)(budget / (int64_t)row_bytes);
  if (stages < 2) return 1;
  if (stages > 8) stages = 8;
  const size_t smem = 128 + (size_t)table_bytes + (size_t)stages * row_bytes;
  int64_t grid = (int64_t)sm_count() * CTAS;
  if (grid > nitems) grid = nitems;
  const bool full = (p.hidden_size >> 3) == THREADS * NVEC;
  const void* fn = full ? reinterpret_cast<const void*>(&scatter_quant_pipe<THREADS, NVEC, true, CTAS>)
                        : reinterpret_cast<const void*>(&scatter_quant_pipe<THREADS, NVEC, false, CTAS>);
  const cudaError_t e = ensure_dynamic_smem(fn, 224 * 1024);
  MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_scatter_quant_i8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  if (full)
    (void)launch_pdl(scatter_quant_pipe<THREADS, NVEC, true, CTAS>, dim3((unsigned)grid), dim3(THREADS), smem, stream, p, stages, table_bytes,
                     pipe_error_ptr());
  else
    (void)launch_pdl(scatter_quant_pipe<THREADS, NVEC, false, CTAS>, dim3((unsigned)grid), dim3(THREADS), smem, stream, p, stages, table_bytes,
                     pipe_error_ptr());
  return check_launch("moe_scatter_quant_i8 (quant, pipelined)");
}

}  // namespace
}  // namespace mcop

using namespace mcop;

extern "C" size_t mcop_moe_scatter_workspace_bytes(int64_t tokens, int topk, int experts_per_rank) {
  if (tokens < 0 || topk < 0 || experts_per_rank < 0) return 0;
  const int64_t tiles = scatter_tiles(tokens);
  // header, [tiles, E] histogram, then the larger of the main path's bitmaps and the general path's ranks
  const int64_t bitmaps = tiles * experts_per_rank * kTileWords, ranks = tokens * topk;
  return (size_t)(64 + tiles * experts_per_rank + (bitmaps > ranks ? bitmaps : ranks)) * sizeof(int32_t);
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
  ScatterWs ws{};
  ws.ticket = reinterpret_cast<int32_t*>(workspace);
  ws.tile_hist = ws.ticket + 64;
  ws.rank = ws.tile_hist + tiles * E;
  if (tokens == 0) {
    cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int32_t) * E, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(starts, 0, sizeof(int32_t) * E, s);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_scatter_quant_i8: memset: %s", cudaGetErrorString(e));
    return MCOP_OK;
  }
  ScatterQuantParams p{};
  p.hidden = reinterpret_cast<const __nv_bfloat16*>(hidden); p.ids = ids; p.weights = weights; p.smooth = smooth;
  p.rows = rows; p.row_scales = row_scales; p.row2tok = row2tok; p.starts = starts; p.counts = counts; p.tok2row = tok2row;
  p.tile_base = ws.tile_hist; p.rank = ws.rank; p.work_counter = ws.ticket + 1;
  p.hist = ws.tile_hist; p.bitmaps = reinterpret_cast<const uint32_t*>(ws.rank);
  p.tokens = tokens; p.hidden_size = (int)hidden_size; p.topk = topk; p.E = E;
  const int nv = (int)(hidden_size >> 3);
  const bool vec_ok = hidden_size % 8 == 0 && aligned16(hidden) && aligned16(smooth) && (reinterpret_cast<uintptr_t>(rows) & 7u) == 0 && nv <= 4096;
  int rc;
  if (vec_ok && nv > 256 && nv <= 2048 && tokens * topk >= 2048) {
    // ---- main path: bitmap kernel + pipelined quant kernel
    const size_t bsmem = (size_t)E * kTileWords * sizeof(uint32_t);
    if (bsmem > 48 * 1024) {
      const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&scatter_bitmap_kernel), bsmem);
      MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_scatter_quant_i8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    (void)launch_pdl(scatter_bitmap_kernel, dim3((unsigned)tiles), dim3(256), bsmem, s, ids, ws.tile_hist, reinterpret_cast<uint32_t*>(ws.rank),
                     ws.ticket + 1, tok2row, tokens, topk, E);
    rc = check_launch("moe_scatter_quant_i8 (bitmaps)");
    if (rc) return rc;
    // a CTA of nv / 4 threads tiles the row exactly (hidden 4096, 5120, 6144, 7168 = 4 x 128 ... 224 vectors of 8):
    // no idle lanes and no bounds tests in the passes, worth 25 % at hidden 7168
    // CTAs of 4 warps whose threads hold 4 to 8 vectors of 8 each tile the usual row lengths exactly (hidden 4096 ... 8192):
    // no idle lanes and no bounds tests in the passes (worth 25 % at hidden 7168), few warps per row barrier, and with
    // 12 to 16 warps per SM enough registers (128 to 168) for the row and the smooth slice of a thread without spills
    if (nv == 896) rc = launch_quant_pipe<128, 7, 3>(p, s);
    else if (nv == 1024) rc = launch_quant_pipe<128, 8, 3>(p, s);
    else if (nv == 768) rc = launch_quant_pipe<128, 6, 3>(p, s);
    else if (nv == 640) rc = launch_quant_pipe<128, 5, 4>(p, s);
    else if (nv == 512) rc = launch_quant_pipe<128, 4, 4>(p, s);
    else if (nv <= 1024) rc = launch_quant_pipe<256, 4, 2>(p, s);
    else rc = launch_quant_pipe<512, 4, 1>(p, s);
    if (rc != 1) return rc;
    // the table of the quant kernel cannot hold this problem: the general path below redoes the counting its own way
  }
  // ---- general path: rank kernel (+ scan kernel), row-per-token quant kernel
  cudaError_t e = cudaMemsetAsync(ws.ticket, 0, 2 * sizeof(int32_t), s);
  MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_scatter_quant_i8: memset: %s", cudaGetErrorString(e));
  const size_t smem = (size_t)E * kTileWords * (sizeof(uint32_t) + sizeof(uint16_t));
  if (smem > 48 * 1024) {
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(&scatter_rank_kernel), smem);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_scatter_quant_i8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  ws.separate_scan = tiles > kInKernelScanTiles;
  scatter_rank_kernel<<<(unsigned)tiles, 256, smem, s>>>(ids, ws, counts, starts, tokens, topk, E);
  rc = check_launch("moe_scatter_quant_i8 (rank)");
  if (rc) return rc;
  if (ws.separate_scan) {
    scatter_scan_kernel<<<(unsigned)E, 256, 0, s>>>(ws, counts, starts, (int)tiles, E);
    rc = check_launch("moe_scatter_quant_i8 (scan)");
    if (rc) return rc;
  }
  const unsigned grid = (unsigned)tokens;
  if (!vec_ok) scatter_quant_any<<<grid, 256, 0, s>>>(p);
  else if (nv <= 256) scatter_quant_vec<128, 2><<<grid, 128, 0, s>>>(p);
  else if (nv <= 1024) scatter_quant_vec<256, 4><<<grid, 256, 0, s>>>(p);
  else if (nv <= 2048) scatter_quant_vec<512, 4><<<grid, 512, 0, s>>>(p);
  else scatter_quant_vec<1024, 4><<<grid, 1024, 0, s>>>(p);
  return check_launch("moe_scatter_quant_i8 (quant)");
}

// ---------------------------------------------------------------------------------------------
// moe_align_block_size: the index preparation of the block-sparse expert GEMM.  The same counting sort as the
// scatter, run over the flat routing entries (a "token" of the rank kernel is one entry, so an expert that a token
// names twice gets two positions), with every expert's range padded to a multiple of block_size.
// ---------------------------------------------------------------------------------------------
extern "C" size_t mcop_moe_align_block_size_workspace_bytes(int64_t numel, int num_experts) {
  if (numel < 0 || num_experts < 0) return 0;
  const int64_t tiles = scatter_tiles(numel);
  return (size_t)(64 + tiles * num_experts + numel + 2 * (int64_t)num_experts) * sizeof(int32_t);
}

extern "C" int mcop_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int num_experts, int block_size,
                                         int32_t* sorted_token_ids, int64_t max_num_tokens_padded, int32_t* expert_ids,
                                         int64_t max_num_blocks, int32_t* num_tokens_post_pad, const int32_t* expert_map,
                                         void* workspace, size_t workspace_bytes, mcop_stream_t stream) {
  MCOP_REQUIRE(sorted_token_ids && expert_ids && num_tokens_post_pad && (topk_ids || numel == 0), MCOP_ERR_ARGUMENT,
               "moe_align_block_size: null pointer");
  MCOP_REQUIRE(numel >= 0 && num_experts >= 1 && max_num_tokens_padded >= 0 && max_num_blocks >= 0, MCOP_ERR_ARGUMENT,
               "moe_align_block_size: bad sizes");
  MCOP_REQUIRE(block_size > 0, MCOP_ERR_ARGUMENT, "moe_align_block_size: block_size should be greater than 0");
  MCOP_REQUIRE(num_experts < kMaxExperts, MCOP_ERR_UNSUPPORTED, "moe_align_block_size: num_experts must be less than %d", kMaxExperts);
  MCOP_REQUIRE(numel + (int64_t)num_experts * block_size <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED,
               "moe_align_block_size: padded positions exceed int32");
  cudaStream_t s = (cudaStream_t)stream;
  if (numel == 0) {  // nothing routed: every position holds the mark numel = 0, no block belongs to an expert
    cudaError_t e = cudaMemsetAsync(sorted_token_ids, 0, sizeof(int32_t) * max_num_tokens_padded, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(expert_ids, 0, sizeof(int32_t) * max_num_blocks, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(num_tokens_post_pad, 0, sizeof(int32_t), s);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_align_block_size: memset: %s", cudaGetErrorString(e));
    return MCOP_OK;
  }
  const size_t need = mcop_moe_align_block_size_workspace_bytes(numel, num_experts);
  MCOP_REQUIRE(workspace && workspace_bytes >= need, MCOP_ERR_WORKSPACE, "moe_align_block_size: workspace of %zu bytes needed, %zu given",
               need, workspace_bytes);
  const int E = num_experts;
  const int64_t tiles = scatter_tiles(numel);
  ScatterWs ws{};
  ws.ticket = reinterpret_cast<int32_t*>(workspace);
  ws.tile_hist = ws.ticket + 64;
  ws.rank = ws.tile_hist + tiles * E;
  int32_t* counts = ws.rank + numel;
  int32_t* starts = counts + E;
  ws.expert_map = expert_map;
  ws.block_size = block_size;
  ws.expert_ids = expert_ids;
  ws.max_blocks = max_num_blocks;
  ws.total = num_tokens_post_pad;
  ws.prefill = sorted_token_ids;
  ws.prefill_n = max_num_tokens_padded;
  ws.prefill_value = (int32_t)numel;
  cudaError_t e = cudaMemsetAsync(ws.ticket, 0, 2 * sizeof(int32_t), s);
  MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_align_block_size: memset: %s", cudaGetErrorString(e));
  const size_t smem = (size_t)E * kTileWords * (sizeof(uint32_t) + sizeof(uint16_t));
  if (smem > 48 * 1024) {
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(&scatter_rank_kernel), smem);
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_align_block_size: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  ws.separate_scan = tiles > kInKernelScanTiles;
  scatter_rank_kernel<<<(unsigned)tiles, 256, smem, s>>>(topk_ids, ws, counts, starts, numel, 1, E);
  int rc = check_launch("moe_align_block_size (rank)");
  if (rc) return rc;
  if (ws.separate_scan) {
    scatter_scan_kernel<<<(unsigned)E, 256, 0, s>>>(ws, counts, starts, (int)tiles, E);
    rc = check_launch("moe_align_block_size (scan)");
    if (rc) return rc;
  }
  align_fill_kernel<<<(unsigned)((numel + 255) / 256), 256, 0, s>>>(topk_ids, ws, starts, sorted_token_ids, numel, E, max_num_tokens_padded);
  return check_launch("moe_align_block_size (fill)");
}
