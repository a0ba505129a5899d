// Part 3c of the hot path: MoE combine (gather).
//
// out[t] (+)= sum over the rows r of token t, in ASCENDING r, of [w(r) *] y[r], accumulated in fp32 and rounded
// once: the result does not depend on scheduling (the reference's bf16 atomics do).
//
// Rows of a token are found through an inverse map: tok2row [tokens, topk] as written by the scatter, or a
// (count, list) table built by a small inversion pre-pass when only the reference's 3-argument signature is
// available.  The main kernel is persistent: a CTA takes chunks of up to 128 consecutive tokens, sorts each token's row
// list in shared memory, and then streams the y rows through a ring of shared-memory stages filled by bulk
// asynchronous copies, so the loads of the rows ahead overlap the adds of the current row.
#include <atomic>

#include "common.cuh"
#include "tma_pipe.cuh"

namespace mcop {
namespace {

struct GatherParams {
  const __nv_bfloat16* y; const int32_t* row2tok; __nv_bfloat16* out;
  const int32_t* tok2row; int topk;                      // direct inverse (nullable)
  const int32_t* head; const int32_t* next;              // inverse built by the pre-pass: per-token chains of row ids
  const int32_t* topk_ids; const float* topk_weights; const int32_t* starts; int experts;  // weighted form
  int64_t rows; int64_t tokens; int hidden_size; int weighted; int accumulate;
};

constexpr int kMaxList = 64;    // rows of one token the row-per-CTA kernels handle without the slow scan
constexpr int kChunkTokens = 64;   // tokens whose row lists a CTA of the pipelined kernel prepares at a time (two such tables + the staging of one)
constexpr int kPipeMaxRows = 16;  // rows per token the pipelined kernel keeps in shared memory

// Inversion pre-pass: the rows of a token form a chain, head[t] -> r1 -> next[r1] -> ... -> -1 (unordered; the gather sorts
// them).  Exact for every distribution of the rows over the tokens: a token of a map with dropped rows may own far more
// rows than rows / tokens, and a table with that average as its width sent such tokens through the scan of the whole map.
// head[] is set to -1 (memset 0xff) before the launch.
__global__ void gather_invert_kernel(const int32_t* __restrict__ row2tok, int32_t* head, int32_t* next, int64_t rows, int64_t tokens) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int t = row2tok[r];
  if (t < 0 || t >= tokens) return;
  next[r] = atomicExch(&head[t], (int32_t)r);
}

// Walks the chain of token t into out[0 .. limit): returns the number of rows, or -1 when there are more than `limit`
// (or the chain is broken: an id outside [0, rows) ends it the same way).
__device__ __forceinline__ int gather_walk_chain(const GatherParams& p, int64_t t, int* out, int limit) {
  int n = 0;
  for (int r = p.head[t]; r >= 0; r = p.next[r]) {
    if (n >= limit || r >= p.rows) return -1;
    out[n++] = r;
  }
  return n;
}

// Weight of row r of token t: the expert owning r is the first e with starts[e+1] > r; the weight is that of
// the first slot of t holding e (0 if none).
__device__ __forceinline__ float row_weight(const GatherParams& p, int64_t t, int64_t r) {
  int lo = 0, hi = p.experts - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (p.starts[mid + 1] > r) hi = mid; else lo = mid + 1;
  }
  for (int j = 0; j < p.topk; ++j)
    if (p.topk_ids[t * p.topk + j] == lo) return p.topk_weights[t * p.topk + j];
  return 0.f;
}

__device__ __forceinline__ void accumulate8(float (&acc)[8], const uint4 raw, bool weighted, float w) {
  float f[8];
  unpack_bf16x8(raw, f);
  if (weighted) {
    // products as packed fp32 pairs (each lane rounded like __fmul_rn), sums scalar: a packed add fed by a packed product
    // would be fused into one multiply-add and drop the product's rounding
    const float2 w2 = make_float2(w, w);
#pragma unroll
    for (int q = 0; q < 8; q += 2) {
      const float2 pr = mul2_rn(make_float2(f[q], f[q + 1]), w2);
      acc[q] = __fadd_rn(acc[q], pr.x);
      acc[q + 1] = __fadd_rn(acc[q + 1], pr.y);
    }
  } else {
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = __fadd_rn(acc[q], f[q]);
  }
}

// Slow path shared by both vector kernels: the token owns more rows than the inverse holds, so row2tok is
// scanned in ascending order.  Every thread walks the same rows; no shared memory, no barrier.
template <int THREADS, int NVEC>
__device__ void accumulate_by_scan(const GatherParams& p, int64_t t, float (&acc)[NVEC][8]) {
  const int nv = p.hidden_size >> 3;
  for (int64_t r = 0; r < p.rows; ++r) {
    if (__ldg(p.row2tok + r) != (int32_t)t) continue;  // uniform over the CTA
    const float w = p.weighted ? row_weight(p, t, r) : 1.f;
    const __nv_bfloat16* src = p.y + r * p.hidden_size;
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
      const int v = threadIdx.x + k * THREADS;
      if (v < nv) accumulate8(acc[k], ld_nc_u4(src + v * 8), p.weighted != 0, w);
    }
  }
}

// Collect the rows of token t in ascending order into s_rows[0..n) (and their weights into s_w).
// Returns n, or -1 if the token has more rows than the inverse holds.
__device__ int gather_collect(const GatherParams& p, int64_t t, int32_t* s_rows, float* s_w, int32_t* s_tmp) {
  __shared__ int s_n;
  int n = 0;
  if (p.tok2row) {
    n = p.topk;
    if (threadIdx.x < n) s_tmp[threadIdx.x] = p.tok2row[t * p.topk + threadIdx.x];
  } else {
    if (threadIdx.x == 0) s_n = gather_walk_chain(p, t, s_tmp, kMaxList);
    __syncthreads();
    n = s_n;
    __syncthreads();  // s_n is reset below
    if (n < 0) return -1;
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
  if (p.weighted && threadIdx.x < n) s_w[threadIdx.x] = row_weight(p, t, s_rows[threadIdx.x]);
  __syncthreads();
  return n;
}

// One CTA per token, rows held in registers.  Used for small problems and for shapes the pipelined kernel
// does not take.
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
            if (v < nv) accumulate8(acc[i], raw[u][i], p.weighted != 0, w);
          }
        }
      }
    }
  } else {
    accumulate_by_scan<THREADS, NVEC>(p, t, acc);
  }
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nv) st_cs_u4(out + v * 8, pack_bf16x8(acc[i]));
  }
}

// One token's ascending row list (and weights) for the pipelined kernel: rows[0..n) and w[0..n), *cnt = n, or -1 when the
// token owns more rows than the table holds (slow scan).  `staged` (nullable): the token's tok2row, ids and weights rows as
// an earlier asynchronous copy left them in shared memory (8 words each, topk <= 8) - the same values as in global memory.
__device__ __forceinline__ void gather_build_list(const GatherParams& p, int64_t t, const uint32_t* staged, int32_t* rows_out, float* w_out,
                                                  int* cnt) {
  int rows[kPipeMaxRows];
  int slot[kPipeMaxRows];  // with tok2row: the routing slot a row came from
  int n = 0;
  bool overflow = false;
  if (p.tok2row) {
    for (int j = 0; j < p.topk; ++j) {
      const int r = staged ? (int)staged[j] : p.tok2row[t * p.topk + j];
      if (r >= 0 && r < p.rows) { rows[n] = r; slot[n] = j; ++n; }
    }
  } else {
    n = gather_walk_chain(p, t, rows, kPipeMaxRows);
    if (n < 0) { overflow = true; n = 0; }
  }
  if (!overflow) {
    for (int a = 1; a < n; ++a) {  // insertion sort, n <= 16
      const int key = rows[a], ks = slot[a];
      int b = a - 1;
      while (b >= 0 && rows[b] > key) { rows[b + 1] = rows[b]; slot[b + 1] = slot[b]; --b; }
      rows[b + 1] = key; slot[b + 1] = ks;
    }
    for (int j = 0; j < n; ++j) {
      rows_out[j] = rows[j];
      if (p.weighted) {
        float w;
        if (p.tok2row) {
          // the row belongs to the expert named by its slot: the weight is that of the FIRST slot of the token that
          // names this expert - the same value the search over the experts' starts would find, without the search
          const int32_t* tid = p.topk_ids + t * p.topk;
          const int e = staged ? (int)staged[8 + slot[j]] : tid[slot[j]];
          int jf = slot[j];
          for (int i = 0; i < slot[j]; ++i)
            if ((staged ? (int)staged[8 + i] : tid[i]) == e) { jf = i; break; }
          w = staged ? __uint_as_float(staged[16 + jf]) : p.topk_weights[t * p.topk + jf];
        } else {
          w = row_weight(p, t, rows[j]);
        }
        w_out[j] = w;
      }
    }
  }
  *cnt = overflow ? -1 : n;
}

// Persistent pipelined kernel.  Dynamic shared memory: 128 bytes of mbarriers, then `stages` row buffers.
// The row lists of a chunk of tokens live in one of two halves of the tables below.  With tok2row and topk <= 8 the
// NEXT chunk's lists are made while the current chunk streams: at the chunk's start one thread per token of the next
// chunk starts asynchronous copies of that token's tok2row, ids and weights rows into shared memory; half way through
// the chunk the same threads wait for their copies (long landed), sort and write the lists into the other half; from
// the next row on the producer runs on into those rows, so the ring neither drains at the chunk's end nor waits for
// three dependent round trips.  Without tok2row (chains to walk) or with more slots the lists are made between chunks.
template <int THREADS, int NVEC>
__global__ void __launch_bounds__(THREADS, (THREADS <= 256 ? 2 : 1)) gather_pipe(GatherParams p, int stages, int chunk, int* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int32_t s_rows[2][kChunkTokens][kPipeMaxRows];
  __shared__ float s_w[2][kChunkTokens][kPipeMaxRows];
  __shared__ int s_cnt[2][kChunkTokens];   // rows of the token; -1 = more than the table holds (slow scan)
  __shared__ uint32_t s_stage[kChunkTokens][24];  // tok2row | ids | weights of the next chunk's tokens, 8 words each
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  unsigned char* buf = smem + 128;
  const int H = p.hidden_size, nv = H >> 3;
  const uint32_t row_bytes = (uint32_t)H * 2u;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();
  pdl_wait();  // nothing of global memory is touched before the kernels ahead in the stream have completed

  uint32_t it = 0;        // items consumed so far by this CTA
  RingPos cons, prod;     // ring positions of the consumer (all threads) and of the producer (thread 0)
  uint32_t issued = 0;    // items issued so far (thread 0 only)
  bool alive = true;
  // every CTA owns one contiguous share of the tokens (equal to within one token, whatever the chunk size) and
  // walks it in chunks
  const int64_t tok_begin = (p.tokens * (int64_t)blockIdx.x) / gridDim.x;
  const int64_t tok_end = (p.tokens * ((int64_t)blockIdx.x + 1)) / gridDim.x;
  const bool ahead = p.tok2row != nullptr && p.topk <= 8;
  uint4 prior[NVEC];  // accumulate: the output row of the token that comes next, as it was before this call
  if (p.accumulate && tok_begin < tok_end) {
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
      const int v = threadIdx.x + k * THREADS;
      if (v < nv) prior[k] = ld_u4(p.out + tok_begin * (int64_t)H + v * 8);
    }
  }
  int cur = 0;
  bool have = false;       // the lists of the chunk at t0 are in half `cur` already
  int qtl = 0, qj = 0;     // thread 0: producer cursor inside the next chunk's lists
  for (int64_t t0 = tok_begin; t0 < tok_end && alive; t0 += chunk) {
    const int ntok = (int)min((int64_t)chunk, tok_end - t0);
    const int nnext = (int)max((int64_t)0, min((int64_t)chunk, tok_end - (t0 + chunk)));
    // ---- phase A: one thread per token builds the token's ascending row list (and weights)
    // (the token's ids and weights prefetched into L1 while its rows are fetched, instead of one round trip after the
    // other: 244 us either way at 32,768 tokens x top-2 - the phase is not what the short runs lose)
    if (!have) {
      if (threadIdx.x < ntok)
        gather_build_list(p, t0 + threadIdx.x, nullptr, s_rows[cur][threadIdx.x], s_w[cur][threadIdx.x], &s_cnt[cur][threadIdx.x]);
      __syncthreads();
    }
    const bool look = ahead && nnext > 0;
    if (look && threadIdx.x < nnext) {
      const int64_t tn = t0 + chunk + threadIdx.x;
      const uint32_t dst = smem_addr(&s_stage[threadIdx.x][0]);
      for (int j = 0; j < p.topk; ++j) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * j), "l"(p.tok2row + tn * p.topk + j) : "memory");
        if (p.weighted) {
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 32u + 4u * j), "l"(p.topk_ids + tn * p.topk + j) : "memory");
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 64u + 4u * j), "l"(p.topk_weights + tn * p.topk + j) : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // ---- phase B: stream the rows of the chunk
    int ptl = 0, pj = 0;  // producer cursor (thread 0)
    if (have) { ptl = qtl; pj = qj; }
    qtl = 0; qj = 0;
    uint32_t ready_after = 0xffffffffu;  // the next chunk's lists may be read once more than this many rows have been consumed
    bool built = false;
    auto issue_next = [&]() -> bool {  // issues the next row of the chunk (or, once listed, of the next chunk), if any
      while (ptl < ntok && (s_cnt[cur][ptl] < 0 || pj >= s_cnt[cur][ptl])) { ++ptl; pj = 0; }
      int32_t row;
      if (ptl < ntok) {
        row = s_rows[cur][ptl][pj++];
      } else {
        if (it <= ready_after) return false;
        while (qtl < nnext && (s_cnt[cur ^ 1][qtl] < 0 || qj >= s_cnt[cur ^ 1][qtl])) { ++qtl; qj = 0; }
        if (qtl >= nnext) return false;
        row = s_rows[cur ^ 1][qtl][qj++];
      }
      const int s = prod.s;
      mbar_expect_tx(&full[s], row_bytes);
      bulk_g2s(buf + (size_t)s * row_bytes, p.y + (int64_t)row * H, row_bytes, &full[s]);
      ++issued;
      prod.advance(stages);
      return true;
    };
    if (threadIdx.x == 0)
      while ((int)(issued - it) < stages)
        if (!issue_next()) break;
    for (int tl = 0; tl < ntok && alive; ++tl) {
      if (look && !built && tl >= ntok / 2) {
        // the next chunk's lists, from the copies started at this chunk's start
        if (threadIdx.x < nnext) {
          asm volatile("cp.async.wait_all;" ::: "memory");
          gather_build_list(p, t0 + chunk + threadIdx.x, s_stage[threadIdx.x], s_rows[cur ^ 1][threadIdx.x], s_w[cur ^ 1][threadIdx.x],
                            &s_cnt[cur ^ 1][threadIdx.x]);
        }
        built = true;
        ready_after = it;  // readable after the next row barrier
      }
      const int64_t t = t0 + tl;
      __nv_bfloat16* out = p.out + t * (int64_t)H;
      float acc[NVEC][8];
#pragma unroll
      for (int k = 0; k < NVEC; ++k) {
        const int v = threadIdx.x + k * THREADS;
        if (p.accumulate && v < nv) {
          unpack_bf16x8(prior[k], acc[k]);
        } else {
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[k][q] = 0.f;
        }
      }
      // accumulate: the NEXT token's output row is asked for now and used one token later (the CTA's tokens are
      // consecutive and only this CTA writes them), instead of a load that the token's first row then waits for
      // (the 3-argument gather, which adds into its output: 205 -> 200 us at 8192 tokens x 8 rows, 2500 us either way at
      // 262,144 tokens x 2 rows = 6.0 TB/s of the 57,344 bytes per token it has to move)
      if (p.accumulate && t + 1 < tok_end) {
#pragma unroll
        for (int k = 0; k < NVEC; ++k) {
          const int v = threadIdx.x + k * THREADS;
          if (v < nv) prior[k] = ld_u4(out + H + v * 8);
        }
      }
      const int n = s_cnt[cur][tl];
      if (n < 0) {
        accumulate_by_scan<THREADS, NVEC>(p, t, acc);
      } else {
        for (int j = 0; j < n; ++j) {
          const int s = cons.s;
          const bool ok = mbar_wait_bounded_sleepy(&full[s], cons.phase, err, 3);
          if (ok) {
            const unsigned char* src = buf + (size_t)s * row_bytes;
            const float w = p.weighted ? s_w[cur][tl][j] : 1.f;
#pragma unroll
            for (int k = 0; k < NVEC; ++k) {
              const int v = threadIdx.x + k * THREADS;
              if (v < nv) accumulate8(acc[k], lds_u4(src + v * 16), p.weighted != 0, w);
            }
          }
          // one barrier per row: agrees on success and tells that every thread has left the stage buffer
          if (!__syncthreads_and(ok)) { alive = false; break; }
          ++it;
          cons.advance(stages);
          if (threadIdx.x == 0) {
            proxy_fence_before_reuse();
            issue_next();
          }
        }
      }
      if (alive) {
#pragma unroll
        for (int k = 0; k < NVEC; ++k) {
          const int v = threadIdx.x + k * THREADS;
          if (v < nv) st_cs_u4(out + v * 8, pack_bf16x8(acc[k]));
        }
      }
    }
    __syncthreads();  // the halves of the tables change hands
    have = look && built;
    cur ^= 1;
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  if (!alive && threadIdx.x == 0) {
    // a wait ran out: drain (bounded) the copies still in flight before the CTA gives its shared memory back
    for (uint32_t k = it; k < issued; ++k, cons.advance(stages))
      (void)mbar_wait_bounded(&full[cons.s], cons.phase, err, 4);
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
        const float w = p.weighted ? row_weight(p, t, r) : 1.f;
        const float f = __bfloat162float(p.y[r * H + i]);
        acc = __fadd_rn(acc, p.weighted ? __fmul_rn(w, f) : f);
      }
    }
    out[i] = __float2bfloat16_rn(acc);
  }
}

// Average rows per token, rounded up and capped: sizes the workspace (tokens * gather_cap >= rows words hold next[]) and
// tells which kernel a map without `tok2row` most likely suits.
int gather_cap(int64_t tokens, int64_t rows) {
  if (tokens <= 0) return 1;
  int64_t c = (rows + tokens - 1) / tokens;
  if (c < 1) c = 1;
  if (c > 32) c = 32;
  return (int)c;
}

template <int THREADS>
int launch_gather_pipe(const GatherParams& p, int64_t tokens, cudaStream_t stream) {
  const size_t row_bytes = (size_t)p.hidden_size * 2;
  // 256-thread CTAs: the ring that still lets two CTAs share an SM beside their tables - with a fixed 96 KB of ring,
  // rows of 6144 and 8192 elements got 8 and 6 stages and ONE CTA per SM: 337 and 367 us at 32,768 tokens x top-2 against
  // 204 and 292 us now (7168: 6 stages and two CTAs either way).  512-thread CTAs are alone on their SM.
  const size_t ring = THREADS <= 256 ? (227 * 1024) / 2 - 24 * 1024 - 128 : 96 * 1024;
  int stages = (int)(ring / row_bytes);
  stages = stages < 2 ? 2 : (stages > 8 ? 8 : stages);
  const size_t smem = 128 + (size_t)stages * row_bytes;
  int per_sm = (int)((227 * 1024) / (smem + 24 * 1024));  // + the static row-list tables and the staging of the next chunk
  per_sm = per_sm < 1 ? 1 : (per_sm > 2048 / THREADS ? 2048 / THREADS : per_sm);
  if (per_sm > 4) per_sm = 4;
  // every CTA gets an equal contiguous share of the tokens and prepares it in chunks of up to kChunkTokens tokens
  int64_t grid = (int64_t)sm_count() * per_sm;
  if (grid > (tokens + 7) / 8) grid = (tokens + 7) / 8;
  // chunks of a quarter of a CTA's share, between 32 and kChunkTokens tokens: with one chunk per CTA every CTA of the
  // grid builds its lists at the same moment and then streams at the same moment (32,768 tokens x top-2, lists made
  // between chunks: 246 us with one chunk of 110 tokens per CTA, 235 / 228 / 239 / 254 us with chunks of 64 / 32 / 16 / 8;
  // with the lists made ahead: 219 / 217 / 220 / 226 / 224 us with chunks of 16 / 24 / 32 / 48 / 64, and no difference
  // beyond the noise at 262,144 tokens)
  const int64_t share = (tokens + grid - 1) / grid;
  int chunk = (int)(((share + 3) / 4 + 7) / 8 * 8);
  chunk = chunk < 32 ? 32 : (chunk > kChunkTokens ? kChunkTokens : chunk);
  const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&gather_pipe<THREADS, 4>), 200 * 1024);
  MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_gather: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  (void)launch_pdl(gather_pipe<THREADS, 4>, dim3((unsigned)grid), dim3(THREADS), smem, stream, p, stages, chunk, pipe_error_ptr());
  return check_launch("moe_gather (pipelined)");
}

int launch_gather(GatherParams p, int64_t tokens, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (tokens == 0) return MCOP_OK;
  MCOP_REQUIRE(tokens <= 0x7fffffffLL && p.rows <= 0x7fffffffLL, MCOP_ERR_UNSUPPORTED, "moe_gather: too many tokens or rows");
  p.tokens = tokens;
  if (p.tok2row) {
    MCOP_REQUIRE(p.topk >= 1 && p.topk <= kMaxList, MCOP_ERR_ARGUMENT, "moe_gather: topk %d out of range with tok2row", p.topk);
  } else {
    const size_t need = mcop_moe_gather_workspace_bytes(tokens, p.rows);
    MCOP_REQUIRE(workspace && workspace_bytes >= need, MCOP_ERR_WORKSPACE, "moe_gather: workspace of %zu bytes needed, %zu given",
                 need, workspace_bytes);
    MCOP_REQUIRE(aligned16(workspace), MCOP_ERR_ARGUMENT, "moe_gather: workspace must be 16-byte aligned");
    int32_t* head = reinterpret_cast<int32_t*>(workspace);
    int32_t* next = head + ((tokens + 63) / 64) * 64;
    p.head = head;
    p.next = next;
    cudaError_t e = cudaMemsetAsync(head, 0xff, (size_t)tokens * sizeof(int32_t), stream);  // every chain empty (-1)
    MCOP_REQUIRE(e == cudaSuccess, MCOP_ERR_CUDA, "moe_gather: memset: %s", cudaGetErrorString(e));
    if (p.rows > 0) {
      const int64_t blocks = (p.rows + 255) / 256;
      gather_invert_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p.row2tok, head, next, p.rows, tokens);
      const int rc = check_launch("moe_gather (invert)");
      if (rc) return rc;
    }
  }
  const int nv = p.hidden_size >> 3;
  const bool vec_ok = p.hidden_size % 8 == 0 && aligned16(p.y) && aligned16(p.out) && nv <= 4096;
  const unsigned grid = (unsigned)tokens;
  const int per_token = p.tok2row ? p.topk : gather_cap(tokens, p.rows);  // without tok2row: the average (a token with more
                                                                         // rows than a kernel's table holds takes the scan)
  // the pipelined kernel pays off once there are a few waves of tokens; rows wider than 2048 vectors or more
  // rows per token than its table holds take the row-per-CTA kernel
  if (vec_ok && nv > 256 && nv <= 2048 && per_token <= kPipeMaxRows && tokens >= 1024) {
    // (CTAs of hidden / 32 threads that tile the row exactly, as the norm and scatter kernels use, measured slower here: 1865
    // against 1745 us at 262,144 tokens x 7168 - the eighth warp is worth more than the idle lanes of the fourth vector)
    if (nv <= 1024) return launch_gather_pipe<256>(p, tokens, stream);
    return launch_gather_pipe<512>(p, tokens, stream);
  }
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

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the inversion table lives in a fixed array inside the library.
// ---------------------------------------------------------------------------------------------
namespace {
// Scratch of mcop_moe_gather_noalloc: the per-token chain heads followed by the per-row links.
// Every device that loads the library holds these 4 MiB until the process exits.
static __device__ __align__(256) int32_t g_gather_noalloc_scratch[MCOP_GATHER_NOALLOC_SCRATCH_BYTES / sizeof(int32_t)];

constexpr int kNoallocMaxDevices = 64;
std::atomic<void*> g_noalloc_ptr[kNoallocMaxDevices];

// Device address of the scratch array on the CURRENT device.  On the host the array's name is only a handle
// of the symbol, not an address a kernel can use, so the address is asked from the runtime, once per device.
void* noalloc_scratch_ptr() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices) {
    set_error(MCOP_ERR_CUDA, "moe_gather_noalloc: cannot identify the current device");
    return nullptr;
  }
  void* p = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (p) return p;
  void* sym = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&sym, g_gather_noalloc_scratch);
  if (e != cudaSuccess || !sym) {
    (void)cudaGetLastError();
    set_error(MCOP_ERR_CUDA, "moe_gather_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    return nullptr;
  }
  g_noalloc_ptr[dev].store(sym, std::memory_order_release);
  return sym;
}
}  // namespace

extern "C" int mcop_moe_gather_noalloc(const void* y, const int32_t* row2tok, void* out, int64_t tokens, int64_t rows,
                                       int64_t hidden_size, mcop_stream_t stream) {
  MCOP_REQUIRE(y && row2tok && out, MCOP_ERR_ARGUMENT, "moe_gather_noalloc: null pointer");
  MCOP_REQUIRE(tokens >= 0 && rows >= 0 && hidden_size > 0 && hidden_size <= 0x7fffffff, MCOP_ERR_ARGUMENT,
               "moe_gather_noalloc: bad sizes");
  const size_t need = mcop_moe_gather_workspace_bytes(tokens, rows);
  MCOP_REQUIRE(need <= MCOP_GATHER_NOALLOC_SCRATCH_BYTES, MCOP_ERR_WORKSPACE,
               "moe_gather_noalloc: %lld tokens x %lld rows need %zu bytes of scratch, the built-in area holds %u; "
               "use mcop_moe_gather with a caller workspace",
               (long long)tokens, (long long)rows, need, (unsigned)MCOP_GATHER_NOALLOC_SCRATCH_BYTES);
  if (tokens == 0) return MCOP_OK;
  void* scratch = noalloc_scratch_ptr();  // first call on this device: resolves the address (not inside a capture)
  if (!scratch) return MCOP_ERR_CUDA;
  GatherParams p{};
  p.y = reinterpret_cast<const __nv_bfloat16*>(y); p.row2tok = row2tok; p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.tok2row = nullptr; p.topk = 0; p.rows = rows; p.hidden_size = (int)hidden_size; p.weighted = 0; p.accumulate = 1;
  // launch_gather resets the chain heads it reads (cudaMemsetAsync on the stream) before the inversion pass, so
  // whatever the previous call left in the array is harmless.
  return launch_gather(p, tokens, scratch, MCOP_GATHER_NOALLOC_SCRATCH_BYTES, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// moe_sum: out[t, :] = sum over the k expert outputs in[t, 0..k-1, :] - the combine step of engines that keep the
// expert outputs token-major ([T, k, H]) instead of scattering them by expert.
// K = 2, 3, 4: running sum kept in T (every partial sum rounded to T, slots in order), as the reference's
// dedicated kernels do; any other k (K = 0): fp32 accumulation in slot order and one rounding, the contract of the
// library reduction the reference falls back to.
// ---------------------------------------------------------------------------------------------
namespace mcop {
namespace {
template <typename T, int K>
__global__ void __launch_bounds__(256) moe_sum_vec(const T* __restrict__ in, T* __restrict__ out, int64_t tokens, int topk, int hidden, float scale) {
  const int nv = hidden >> 3;
  const int64_t total = tokens * nv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / nv;
    const int v = (int)(i - t * nv);
    const T* src = in + (t * topk) * (int64_t)hidden + v * 8;
    float acc[8];
    if constexpr (K > 0) {
      float x[K][8];
#pragma unroll
      for (int k = 0; k < K; ++k) Vec8<T>::load_nc(src + (int64_t)k * hidden, x[k]);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = x[0][j];
#pragma unroll
      for (int k = 1; k < K; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = round_to<T>(__fadd_rn(acc[j], x[k][j]));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 4
      for (int k = 0; k < topk; ++k) {
        float x[8];
        Vec8<T>::load_nc(src + (int64_t)k * hidden, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], x[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fmul_rn(acc[j], scale);  // 1 for moe_sum (exact), the routed scaling factor for moe_sum_reduce
    }
    Vec8<T>::store(out + t * (int64_t)hidden + v * 8, acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_sum_any(const T* __restrict__ in, T* __restrict__ out, int64_t tokens, int topk, int hidden,
                                                   float scale, int per_add_form) {
  const int64_t total = tokens * hidden;
  const bool per_add = per_add_form && topk >= 2 && topk <= 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / hidden;
    const int c = (int)(i - t * hidden);
    const T* src = in + (t * topk) * (int64_t)hidden + c;
    float acc = per_add ? ElemTraits<T>::to_float(src[0]) : 0.f;
    for (int k = per_add ? 1 : 0; k < topk; ++k) {
      acc = __fadd_rn(acc, ElemTraits<T>::to_float(src[(int64_t)k * hidden]));
      if (per_add) acc = round_to<T>(acc);
    }
    if (!per_add) acc = __fmul_rn(acc, scale);
    out[i] = ElemTraits<T>::from_float(acc);
  }
}

template <typename T>
int launch_moe_sum(const void* input, void* output, int64_t tokens, int topk, int64_t hidden, float scale, bool per_add_form,
                   cudaStream_t stream) {
  const T* in = reinterpret_cast<const T*>(input);
  T* out = reinterpret_cast<T*>(output);
  const bool vec_ok = hidden % 8 == 0 && aligned16(input) && aligned16(output);
  const int64_t work = vec_ok ? tokens * (hidden >> 3) : tokens * hidden;
  int64_t grid = (work + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;  // grid-stride beyond a few waves of resident CTAs
  if (grid > cap) grid = cap;
  const int H = (int)hidden;
  if (!vec_ok) moe_sum_any<T><<<(unsigned)grid, 256, 0, stream>>>(in, out, tokens, topk, H, scale, per_add_form ? 1 : 0);
  else if (per_add_form && topk == 2) moe_sum_vec<T, 2><<<(unsigned)grid, 256, 0, stream>>>(in, out, tokens, topk, H, scale);
  else if (per_add_form && topk == 3) moe_sum_vec<T, 3><<<(unsigned)grid, 256, 0, stream>>>(in, out, tokens, topk, H, scale);
  else if (per_add_form && topk == 4) moe_sum_vec<T, 4><<<(unsigned)grid, 256, 0, stream>>>(in, out, tokens, topk, H, scale);
  else moe_sum_vec<T, 0><<<(unsigned)grid, 256, 0, stream>>>(in, out, tokens, topk, H, scale);
  return check_launch("moe_sum");
}
}  // namespace
}  // namespace mcop

static int moe_sum_entry(const char* name, const void* input, void* output, int64_t tokens, int topk, int64_t hidden_size, float scale,
                         bool per_add_form, int dtype, mcop_stream_t stream) {
  MCOP_REQUIRE(input && output, MCOP_ERR_ARGUMENT, "%s: null pointer", name);
  MCOP_REQUIRE(tokens >= 0 && topk >= 1 && hidden_size > 0 && hidden_size <= 0x7fffffff, MCOP_ERR_ARGUMENT, "%s: bad sizes", name);
  if (tokens == 0) return MCOP_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == MCOP_BF16) return launch_moe_sum<__nv_bfloat16>(input, output, tokens, topk, hidden_size, scale, per_add_form, s);
  if (dtype == MCOP_F16) return launch_moe_sum<__half>(input, output, tokens, topk, hidden_size, scale, per_add_form, s);
  if (dtype == MCOP_F32) return launch_moe_sum<float>(input, output, tokens, topk, hidden_size, scale, per_add_form, s);
  return set_error(MCOP_ERR_UNSUPPORTED, "%s: dtype %d", name, dtype);
}

extern "C" int mcop_moe_sum(const void* input, void* output, int64_t tokens, int topk, int64_t hidden_size, int dtype,
                            mcop_stream_t stream) {
  return moe_sum_entry("moe_sum", input, output, tokens, topk, hidden_size, 1.0f, true, dtype, stream);
}

// sglang's moe_sum_reduce (op/sglang/csrc/moe/moe_sum_reduce.cu:119-223): fp32 accumulation in slot order for every topk,
// times the routed scaling factor (as float), one rounding.
extern "C" int mcop_moe_sum_reduce(const void* input, void* output, int64_t tokens, int topk, int64_t hidden_size,
                                   double routed_scaling_factor, int dtype, mcop_stream_t stream) {
  return moe_sum_entry("moe_sum_reduce", input, output, tokens, topk, hidden_size, (float)routed_scaling_factor, false, dtype, stream);
}
