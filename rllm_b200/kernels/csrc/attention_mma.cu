// Paged causal attention for bfloat16 on tensor cores (mma.sync m16n8k16,
// float32 accumulate), grouped-query aware: the query heads that share a kv
// head are packed into the rows of one tile, so a K/V tile is loaded once for
// all of them.
//
//   prefill kernel  rows = (query token, head of the group); 4 warps x 16 rows;
//                   key tiles of 64, double-buffered with cp.async; online
//                   softmax in float32 (FlashAttention-2 schedule).
//   decode kernel   one query token per sequence; a warp walks a 128-key chunk
//                   of one (sequence, kv head) in tiles of 32 with its own
//                   cp.async pipeline and online softmax; partial (max, sum,
//                   output) go to a workspace and the last warp of a sequence
//                   merges its chunks in order.  The token's rotation and
//                   cache write can be fused in.
//
// Contract as in attention_simt.cu: the query at position p of sequence s
// sees keys max(0, p - window + 1) .. p (window 0: all), read from the cache
// through the block table; kv head of head h is h / (nq / nkv); scores are
// scaled by `scale`; softmax and both accumulations are float32.  Key tiles and
// splits are aligned to absolute positions (multiples of 32, 64 and 128), so a
// row's arithmetic does not depend on the batch around it or on how its
// sequence was cut into steps.
//
// The reference's kernels for the same job are one-thread-per-element CUDA-core
// loops (crates/rllm-kernels/src/cuda/paged_attention.cu:88-179, 252-347).
#include "common.cuh"
#include <stdlib.h>
#include <math.h>

#define BM 64          // rows per CTA (prefill)
#define BN 64          // keys per tile
#define NTHREADS 128

__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;   // n = 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(unsigned*)&v;
}

// A tile is [rows][D] bf16; its 16-byte chunks are XOR-swizzled so that the 8
// rows an ldmatrix reads fall into 8 different bank groups.
template <int D> __device__ __forceinline__ int swz(int row, int chunk) {
  constexpr int C = D / 8;
  if (C >= 8) return chunk ^ (row & 7);
  if (C == 4) return chunk ^ ((row >> 1) & 3);
  return chunk ^ ((row >> 2) & 1);
}
template <int D> __device__ __forceinline__ bf16* tile_ptr(bf16* base, int row, int chunk) {
  return base + row * D + swz<D>(row, chunk) * 8;
}

// Where the keys j0 .. j0+rows-1 of one kv head of a sequence lie in the paged
// cache: element offset of each key's row (the same in the K and the V cache),
// or -1 for keys outside [lo, hi) and for pages the sequence does not hold.
// Called by `rows` threads (one key each); the caller synchronises before the
// offsets are used.
__device__ __forceinline__ void kv_row_offsets(long long* rowoff, const int* __restrict__ bt, int j0, int r,
                                               int lo, int hi, int kvh, int nkv, int page_size, int page_shift,
                                               int num_pages, int D, int* err) {
  const int j = j0 + r;
  long long off = -1;
  if (j >= lo && j < hi) {
    const int pi = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
    const int pr = page_shift >= 0 ? (j & (page_size - 1)) : (j - pi * page_size);
    const int page = bt[pi];
    if (page < 0 || page >= num_pages) atomicOr(err, 4);
    else off = (((long long)page * nkv + kvh) * page_size + pr) * D;
  }
  rowoff[r] = off;
}

// Copy `rows` key rows of K and of V from the caches into two swizzled tiles;
// rows with offset -1 are zero-filled.  A thread keeps one 16-byte column and
// walks down the rows, rstep at a time; its swizzled column takes two values.
template <int D>
__device__ __forceinline__ void copy_kv_pair(bf16* tile_k, bf16* tile_v, const bf16* __restrict__ kcache,
                                             const bf16* __restrict__ vcache, const long long* rowoff,
                                             int rows, int tid, int nthreads) {
  constexpr int C = D / 8;
  const int c = tid % C;
  const int rstep = nthreads / C;          // nthreads is a multiple of C (C <= 16, nthreads >= 32)
  const bf16* kcol = kcache + c * 8;
  const bf16* vcol = vcache + c * 8;
#pragma unroll 4
  for (int r = tid / C; r < rows; r += rstep) {
    const long long off = rowoff[r];
    const bool ok = off >= 0;
    const int d = r * D + swz<D>(r, c) * 8;
    cp_async16(tile_k + d, ok ? kcol + off : kcache, ok);
    cp_async16(tile_v + d, ok ? vcol + off : vcache, ok);
  }
}

// S[16 x 8 NT] = Q_frag . K_tile^T for one warp; accumulators s[NT n-tiles][4].
template <int D, int NT>
__device__ __forceinline__ void qk_tile(float (*s)[4], const unsigned (*qf)[4], bf16* sK, int lane) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {   // two n-tiles (16 keys) per ldmatrix.x4
      const int mat = lane >> 3;
      const int key = np * 16 + (lane & 7) + (mat >> 1) * 8;
      const int chunk = kk * 2 + (mat & 1);
      unsigned b0, b1, b2, b3;
      ldmatrix_x4(b0, b1, b2, b3, tile_ptr<D>(sK, key, chunk));
      mma_bf16(s[np * 2], qf[kk], b0, b1);
      mma_bf16(s[np * 2 + 1], qf[kk], b2, b3);
    }
  }
}

// O[16 x D] += P[16 x 8 NT] . V_tile for one warp; p given as accumulators.
template <int D, int NT>
__device__ __forceinline__ void pv_tile(float (*o)[4], const float (*p)[4], bf16* sV, int lane) {
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {     // 16 keys per k-step
    unsigned a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {   // two n-tiles (16 dims) per ldmatrix.x4.trans
      const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int chunk = dp * 2 + (lane >> 4);
      unsigned b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, tile_ptr<D>(sV, key, chunk));
      mma_bf16(o[dp * 2], a, b0, b1);
      mma_bf16(o[dp * 2 + 1], a, b2, b3);
    }
  }
}

// Online-softmax update of one warp's 16 x (8 NT) score tile.  Thread holds rows
// r0 = lane/4 and r0 + 8; positions and key ranges per row are given.
//   s: raw scores in, probabilities out;  m, l: running max (log2 domain) and sum.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));   // ex2(-inf) = +0
  return y;
}

template <int DT, int NT>
__device__ __forceinline__ void softmax_tile(float (*s)[4], float (*o)[4], float* m, float* l, int j0,
                                             const int* row_lo, const int* row_hi, float scale_log2,
                                             int lane) {
  const bool whole = j0 >= row_lo[0] && j0 + NT * 8 <= row_hi[0] && j0 >= row_lo[1] && j0 + NT * 8 <= row_hi[1];
  if (!__all_sync(0xffffffffu, whole)) {     // some key of this tile is masked for some row of the warp
    const int col0 = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int hrow = e >> 1;
        const int j = j0 + nt * 8 + col0 + (e & 1);
        if (!(j >= row_lo[hrow] && j < row_hi[hrow])) s[nt][e] = -INFINITY;
      }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
  }
  // scores are scaled here (scale_log2 > 0): max of the raw scores times the scale
  float corr[2], msafe[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float mnew = fmaxf(m[h], mx[h] * scale_log2);
    msafe[h] = (mnew == -INFINITY) ? 0.f : mnew;        // a row that has seen nothing yet
    corr[h] = ex2_approx(m[h] - msafe[h]);              // m = -inf gives 0; its sums are 0 anyway
    m[h] = mnew;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int hrow = e >> 1;
      const float p = ex2_approx(fmaf(s[nt][e], scale_log2, -msafe[hrow]));   // a masked score gives 0
      s[nt][e] = p;
      sum[hrow] += p;
    }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
    sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
    l[h] = l[h] * corr[h] + sum[h];
  }
  if (!__all_sync(0xffffffffu, corr[0] == 1.f && corr[1] == 1.f)) {   // the max of some row moved
#pragma unroll
    for (int nt = 0; nt < DT; ++nt) {
      o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
      o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
    }
  }
}

// ---------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(NTHREADS, (D <= 64 ? 4 : 2))
attention_prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out,
                         const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                         const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ q_start, const int* __restrict__ seq_lens, int seq_begin,
                         int seq_end, int nq, int nkv, int page_size, int num_pages, int window,
                         float scale_log2, int* __restrict__ err) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* sQ = (bf16*)smem_raw;          // [BM][D]
  bf16* sK = sQ + BM * D;              // 2 stages [BN][D]
  bf16* sV = sK + 2 * BN * D;          // 2 stages [BN][D]
  long long* sOff = (long long*)(sV + 2 * BN * D);   // 2 stages [BN] row offsets
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = nq / nkv;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  const int bq = BM / g;               // query tokens per tile (rows beyond bq * g stay idle)
  const int kvh = blockIdx.x % nkv;
  // which (sequence, tile) is this CTA?
  // CTAs are handed out in order of blockIdx: the last tiles of a sequence see the most keys, so
  // they get the lowest indices (for every kv head) and start first
  int s = -1, tile = 0;
  {
    int left = blockIdx.x / nkv;
    for (int i = seq_begin; i < seq_end; ++i) {
      const int n = (q_start[i + 1] - q_start[i] + bq - 1) / bq;
      if (left < n) { s = i; tile = n - 1 - left; break; }
      left -= n;
    }
  }
  if (s < 0) return;
  const int qs = q_start[s], qlen = q_start[s + 1] - qs;
  const int pos0 = seq_lens[s] - qlen;         // position of the sequence's first query token
  const int t0 = tile * bq;                    // first query token of the tile (within this step)
  const int ntok = min(bq, qlen - t0);
  const int* bt = block_table + (size_t)s * max_blocks;

  // Q tile: row r = token (t0 + r / g), head (kvh * g + r % g)
  {
    constexpr int C = D / 8;
    for (int idx = tid; idx < BM * C; idx += NTHREADS) {
      const int r = idx / C, c = idx - r * C;
      const int tl = r / g, hl = r - tl * g;
      const bool ok = tl < ntok;
      const bf16* src = ok ? q + (size_t)(qs + t0 + tl) * q_stride + (size_t)(kvh * g + hl) * D + c * 8 : q;
      cp_async16(tile_ptr<D>(sQ, r, c), src, ok);
    }
  }
  cp_async_commit();

  const int first_pos = pos0 + t0, last_pos = pos0 + t0 + ntok - 1;
  const int kmin = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
  const int kend = last_pos + 1;
  const int tile_lo = kmin / BN, tile_hi = (kend + BN - 1) / BN;

  // this thread's two rows
  int row_lo[2], row_hi[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int tl = r / g;
    if (tl < ntok) {
      const int p = pos0 + t0 + tl;
      row_hi[h] = p + 1;
      row_lo[h] = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    } else {
      row_lo[h] = 0; row_hi[h] = 0;            // idle row: sees nothing
    }
  }

  if (tid < BN) kv_row_offsets(sOff, bt, tile_lo * BN, tid, kmin, kend, kvh, nkv, page_size, page_shift, num_pages, D, err);
  __syncthreads();
  copy_kv_pair<D>(sK, sV, kcache, vcache, sOff, BN, tid, NTHREADS);
  cp_async_commit();

  cp_async_wait<1>();      // Q has landed
  __syncthreads();
  unsigned qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int row = warp * 16 + (lane & 15);
    const int chunk = kk * 2 + (lane >> 4);
    ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], tile_ptr<D>(sQ, row, chunk));
  }

  float o[D / 8][4];
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int kt = tile_lo; kt < tile_hi; ++kt) {
    const int stage = (kt - tile_lo) & 1;
    const bool more = kt + 1 < tile_hi;
    if (more && tid < BN)
      kv_row_offsets(sOff + (stage ^ 1) * BN, bt, (kt + 1) * BN, tid, kmin, kend, kvh, nkv, page_size, page_shift,
                     num_pages, D, err);
    cp_async_wait<0>();
    __syncthreads();       // this stage's K and V are in; the next stage's offsets are published
    if (more) {            // the other stage was last read before the barrier that ended the previous iteration
      copy_kv_pair<D>(sK + (stage ^ 1) * BN * D, sV + (stage ^ 1) * BN * D, kcache, vcache,
                      sOff + (stage ^ 1) * BN, BN, tid, NTHREADS);
      cp_async_commit();
    }
    float sc[8][4];
    qk_tile<D, 8>(sc, qf, sK + stage * BN * D, lane);
    softmax_tile<D / 8, 8>(sc, o, m, l, kt * BN, row_lo, row_hi, scale_log2, lane);
    pv_tile<D, 8>(o, sc, sV + stage * BN * D, lane);
    __syncthreads();
  }

  // epilogue: O / l
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int tl = r / g, hl = r - tl * g;
    if (tl >= ntok) continue;
    const float inv = l[h] > 0.f ? 1.0f / l[h] : 0.f;
    bf16* orow = out + ((size_t)(qs + t0 + tl) * nq + kvh * g + hl) * D + (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      __nv_bfloat162 v = __floats2bfloat162_rn(o[nt][h * 2] * inv, o[nt][h * 2 + 1] * inv);
      *(__nv_bfloat162*)(orow + nt * 8) = v;
    }
  }
}

// ---------------------------------------------------------------------------
// decode: one query token per sequence.  The keys of a (sequence, kv head) are
// cut into chunks of 128 at absolute positions; one warp takes one chunk and
// walks it in tiles of 32 keys with its own cp.async pipeline and an online
// softmax in registers.  Warps are independent; a CTA is just 1, 2 or 4 of
// them.  Every chunk leaves its partial (max, sum, output) in the workspace; the
// CTA that finds itself last for its (sequence, kv head) merges all chunks in
// order, so the result does not depend on the CTA shape, the pipeline depth or
// the batch.  Optionally fused in: the rotation of the token's q and k
// (rotate-half over the first rotary_dim dims, angle position * f_i reduced in
// float64, cosine and sine in float32) and the write of its k and v into their
// cache page.
// Workspace (floats): partial outputs [S, nq, max_chunks, D], then (max, sum)
// pairs [S, nq, max_chunks, 2].  Counters: int [S * nkv], zero before the call;
// the kernel leaves them zero.
// ---------------------------------------------------------------------------
#define CHUNK 128        // keys per chunk (= per warp) at most; walked in tiles of TBN = 32 or 16 keys
// A sequence's chunks have 64 keys instead where the launch allows it (small_below > 0) and the work is small:
// where sequences x kv heads x ceil(length / 128) stays below small_below, twice as many warps walk half as
// many tiles one after the other, and the chain load - scores - softmax - product that a warp goes through for
// each of its tiles is half as long (batch 8 at 2,304 keys in a decode step: +5 % tokens a second end to end,
// batch 1: +3 %; at 4,096 keys and batch 8, or at batch 64, chunks of 128 are ahead by 3 to 4 %).  The rule
// looks at the sequence's own length, so that a sequence's result depends on the number of sequences beside
// it only through the order in which partial results are added.
#define CHUNK_SMALL 64
#define CHUNK_SMALL_BELOW 1536

// a warp's shared memory: STAGES x (K tile, V tile), the Q tile [16][D], the cache row of each of the
// chunk's keys, cosines and sines
template <int D, int STAGES, int TBN> __host__ __device__ constexpr int dec_warp_smem() {
  return STAGES * 2 * TBN * D * 2 + 16 * D * 2 + CHUNK * 4 + (D < 32 ? 32 : D) * 4;
}

// Copy `rows` key rows of K and of V (cache row numbers in rowidx, -1: zero-fill) into two swizzled tiles.
template <int D>
__device__ __forceinline__ void copy_kv_rows(bf16* tile_k, bf16* tile_v, const bf16* __restrict__ kcache,
                                             const bf16* __restrict__ vcache, const int* rowidx, int rows, int lane) {
  constexpr int C = D / 8;
  const int c = lane % C;
  constexpr int rstep = 32 / C;
  const bf16* kcol = kcache + c * 8;
  const bf16* vcol = vcache + c * 8;
#pragma unroll 4
  for (int r = lane / C; r < rows; r += rstep) {
    const int row = rowidx[r];
    const bool ok = row >= 0;
    const long long off = (long long)row * D;
    const int d = r * D + swz<D>(r, c) * 8;
    cp_async16(tile_k + d, ok ? kcol + off : kcache, ok);
    cp_async16(tile_v + d, ok ? vcol + off : vcache, ok);
  }
}

// The same for a tile whose `rows` keys are all to be read and lie in one page (split = rows) or in two
// (the first `split` in the page whose first cache row is row_a, the rest from row_b on): a page's rows follow one
// another in the cache, so a lane needs one pointer a page and constant steps from it, where the general form
// looks every row up (stamped with heads of 128: 800 cycles a tile of 16 keys for the general form, of 1,900).
template <int D, int ROWS>
__device__ __forceinline__ void copy_kv_pages(bf16* tile_k, bf16* tile_v, const bf16* __restrict__ kcache,
                                              const bf16* __restrict__ vcache, int row_a, int row_b, int split, int lane) {
  constexpr int C = D / 8;
  constexpr int rstep = 32 / C;
  const int c = lane % C, r0 = lane / C;
  const long long oa = (long long)row_a * D + c * 8, ob = (long long)(row_b - split) * D + c * 8;
#pragma unroll
  for (int i = 0; i < ROWS / rstep; ++i) {
    const int r = r0 + i * rstep;
    const long long off = ((i * rstep >= split) ? ob : oa) + (long long)r * D;      // (split is a multiple of rstep)
    const int d = r * D + swz<D>(r, c) * 8;
    cp_async16(tile_k + d, kcache + off, true);
    cp_async16(tile_v + d, vcache + off, true);
  }
}

// SMALL: the smaller chunks are an option (small_below > 0) and the grid is laid out for them; without it the
// chunk size is a constant of the kernel, which then is the kernel it was (registers and all).
template <int D, int STAGES, int TBN, bool SMALL>
__global__ void __launch_bounds__(128, (STAGES == 1 && D <= 64 ? 5 : 1))
attention_decode_kernel(bf16* __restrict__ qkv, int q_stride, bf16* __restrict__ out,
                        bf16* __restrict__ kcache, bf16* __restrict__ vcache,
                        const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ seq_lens, int nq, int nkv, int page_size, int num_pages,
                        int window, float scale_log2, int max_chunks, const double* __restrict__ inv_freq,
                        int rotary_dim, int write_kv, float* __restrict__ ws_o, float* __restrict__ ws_ml,
                        int* __restrict__ counters, int* __restrict__ err, int tail_from, int first_wave,
                        int small_below) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char* mine = smem_raw + (size_t)warp * dec_warp_smem<D, STAGES, TBN>();
  bf16* sW = (bf16*)mine;                                          // STAGES x (K [32][D], V [32][D])
  bf16* sQ = sW + STAGES * 2 * TBN * D;                         // [16][D]
  int* sRowIdx = (int*)(sQ + 16 * D);                              // [CHUNK] cache row of each key of the chunk
  float* sCS = (float*)(sRowIdx + CHUNK);                          // cos[D/2], sin[D/2]
  // With write_kv nothing that this kernel reads before the wait below was written by the kernel
  // before it in the stream: lengths and block tables are inputs of the step, the cache rows of
  // earlier positions are from earlier steps (the token's own key and value come from qkv, after
  // the wait).  So the first tiles are on their way while that kernel finishes.  Without write_kv
  // the token's key was stored by the kernel before this one: wait first.
  if (!write_kv) pdl_wait();
  const int g = nq / nkv;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  // Grid (CTAs of a sequence, kv heads, sequences), or, where the smaller chunks are an option, (kv heads,
  // sequences, CTAs of a sequence): CTAs start in the order of their linear index, x first, so in the second
  // form the CTAs whose chunks lie behind a short sequence's end (the grid is made for the longest allowed,
  // in the smaller chunks) come last and keep no CTA with work out of the first wave (batch 8 at 4,092 keys:
  // 7 % of a decode step); with many sequences the first form is 4 % ahead (a sequence's CTAs run, end and
  // are merged together).
  constexpr bool seq_major = !SMALL;
  const int cta_x = seq_major ? blockIdx.x : blockIdx.z;
  const int kvh = seq_major ? blockIdx.y : blockIdx.x, s = seq_major ? blockIdx.z : blockIdx.y;
  const int chunk = cta_x * (blockDim.x >> 5) + warp;
  const int len = seq_lens[s];
  const int pos = len - 1;
  const int kmin = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int ck = (SMALL && (long long)gridDim.x * gridDim.y * ((len + CHUNK - 1) / CHUNK) < small_below) ? CHUNK_SMALL : CHUNK;   // (SMALL: x, y = kv heads, sequences)
  const int w0 = chunk * ck;
  const int nwarps = blockDim.x >> 5;
  {  // a CTA none of whose chunks holds a visible key has nothing to do
    const int first = cta_x * nwarps * ck;
    if (first >= len || first + nwarps * ck <= kmin) {
      // It still waits for the kernel ahead (it has not yet, with write_kv): a CTA that exits counts as
      // having let the next kernel in, and that kernel may then assume that everything but this kernel is
      // complete.  These CTAs do no work, so the wait costs nothing.
      if (write_kv) pdl_wait();
      return;
    }
  }
  const bool active = w0 < len && w0 + ck > kmin;
  const int* bt = block_table + (size_t)s * max_blocks;
  const int half = rotary_dim >> 1;
  bf16* qrow = qkv + (size_t)s * q_stride;
  // keys to read from the cache: with write_kv the token's own key comes from qkv, not from the cache
  const int read_hi = write_kv ? pos : len;
  const int t_lo = active ? (kmin > w0 ? (kmin - w0) / TBN : 0) : 0;
  const int t_hi = active ? min((ck / TBN), (len - w0 + TBN - 1) / TBN) : 0;

  // where the chunk's keys lie: all block-table lookups at once
  if (active) {
#pragma unroll
    for (int i = 0; i < CHUNK / 32; ++i) {
      if (i * 32 >= ck) break;
      const int j = w0 + i * 32 + lane;
      int row = -1;
      if (j >= kmin && j < read_hi) {
        const int pi = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
        const int pr = page_shift >= 0 ? (j & (page_size - 1)) : (j - pi * page_size);
        const int page = bt[pi];
        if (page < 0 || page >= num_pages) atomicOr(err, 4);
        else row = (page * nkv + kvh) * page_size + pr;
      }
      sRowIdx[i * 32 + lane] = row;
    }
  }
  __syncwarp();
  // tiles that lie in one page, or in two whole pages, and are read whole take the short way
  const int split = page_size < TBN ? page_size : TBN;
  const bool by_pages = page_shift >= 0 && (page_size % TBN == 0 || TBN == 2 * page_size) && split % (32 / (D / 8)) == 0;
  auto issue = [&](int t) {
    if (t < t_hi) {
      bf16* st = sW + ((t - t_lo) % STAGES) * 2 * TBN * D;
      const int j0 = w0 + t * TBN;
      const int row_a = sRowIdx[t * TBN], row_b = sRowIdx[t * TBN + (split < TBN ? split : 0)];
      if (by_pages && j0 >= kmin && j0 + TBN <= read_hi && row_a >= 0 && row_b >= 0)
        copy_kv_pages<D, TBN>(st, st + TBN * D, kcache, vcache, row_a, row_b, split, lane);
      else
        copy_kv_rows<D>(st, st + TBN * D, kcache, vcache, sRowIdx + t * TBN, TBN, lane);
    }
    cp_async_commit();
  };
  // Q rows = heads of the group, rows >= g zero: 16-byte loads into registers.  The loads take as long as a
  // tile's, so they go out before the first tiles are asked for wherever the kernel ahead in the stream is
  // through anyway: without write_kv (waited for above), and in CTAs behind the grid's first wave, which
  // start when CTAs of this grid have finished (if that kernel should still run, they wait here, no more).
  // A CTA of the first wave starts while that kernel runs: it asks for its tiles first and waits then.
  // (The row is the output of the kernel ahead: it is read through a pointer made behind the wait, so that no
  // load of it can be merged with another or moved above the wait; see pdl_fresh.)
  constexpr int QN = 16 * (D / 8) / 32;
  uint4 qreg[QN];
  const bf16* qrow_now = nullptr;
  auto load_q = [&]() {
    qrow_now = pdl_fresh((const bf16*)qrow);
#pragma unroll
    for (int i = 0; i < QN; ++i) {
      const int idx = lane + 32 * i, r = idx / (D / 8), c = idx % (D / 8);
      qreg[i] = r < g ? *(const uint4*)(qrow_now + (size_t)(kvh * g + r) * D + c * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  const int cta_id = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
  const bool q_first = !write_kv || cta_id >= first_wave;
  if (q_first) {
    if (write_kv) pdl_wait();
    load_q();
  }
#pragma unroll
  for (int i = 0; i < STAGES; ++i) issue(t_lo + i);
  // the rotation's angles depend on the position alone
  for (int i = lane; i < half; i += 32) rope_cos_sin(pos, inv_freq[i], &sCS[i], &sCS[half + i]);
  if (!q_first) {
    pdl_wait();
    load_q();
  }
  // no CTA of this grid is still to come once its last wave runs: the stream's next kernel may come in
  if (cta_id >= tail_from) pdl_launch();

  // the Q tile in shared memory, then the rotation there (a lane rotates the pairs (i, i + half) it owns)
#pragma unroll
  for (int i = 0; i < QN; ++i) {
    const int idx = lane + 32 * i, r = idx / (D / 8), c = idx % (D / 8);
    *(uint4*)tile_ptr<D>(sQ, r, c) = qreg[i];
  }
  __syncwarp();
  for (int idx = lane; idx < g * half; idx += 32) {
    const int r = idx / half, i = idx - r * half;
    bf16* pa = tile_ptr<D>(sQ, r, i >> 3) + (i & 7);
    bf16* pb = tile_ptr<D>(sQ, r, (i + half) >> 3) + ((i + half) & 7);
    const float a = to_f32(*pa), b = to_f32(*pb);
    const float cs = sCS[i], sn = sCS[half + i];
    *pa = from_f32<bf16>(a * cs - b * sn);
    *pb = from_f32<bf16>(b * cs + a * sn);
  }
  __syncwarp();

  float o[D / 8][4];
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  {
    unsigned qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], tile_ptr<D>(sQ, lane & 15, kk * 2 + (lane >> 4)));
    int row_lo[2], row_hi[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = (lane >> 2) + h * 8;
      row_lo[h] = kmin;
      row_hi[h] = r < g ? len : 0;
    }
    for (int t = t_lo; t < t_hi; ++t) {
      bf16* sK = sW + ((t - t_lo) % STAGES) * 2 * TBN * D;
      bf16* sV = sK + TBN * D;
      cp_async_wait<STAGES - 1>();
      __syncwarp();
      const int j0 = w0 + t * TBN;
      if (write_kv && pos >= j0 && pos < j0 + TBN) {
        // the token's own k (rotated) and v: into the cache page, and into this tile
        const int pi = page_shift >= 0 ? (pos >> page_shift) : (pos / page_size);
        const int page = bt[pi];
        const bool okp = page >= 0 && page < num_pages;
        if (!okp && lane == 0) atomicOr(err, 2);
        const long long off = (((long long)(okp ? page : 0) * nkv + kvh) * page_size + (pos - pi * page_size)) * D;
        const bf16* kx = qrow_now + (size_t)(nq + kvh) * D;
        const bf16* vx = qrow_now + (size_t)(nq + nkv + kvh) * D;
        const int r = pos - j0;
        for (int i = lane; i < D; i += 32) {
          float kv = to_f32(kx[i]);
          if (i < half) kv = kv * sCS[i] - to_f32(kx[i + half]) * sCS[half + i];
          else if (i < rotary_dim) kv = kv * sCS[i - half] + to_f32(kx[i - half]) * sCS[i];
          const bf16 kb = from_f32<bf16>(kv), vb = vx[i];
          tile_ptr<D>(sK, r, i >> 3)[i & 7] = kb;
          tile_ptr<D>(sV, r, i >> 3)[i & 7] = vb;
          if (okp) { kcache[off + i] = kb; vcache[off + i] = vb; }
        }
        __syncwarp();
      }
      float sc[TBN / 8][4];
      qk_tile<D, TBN / 8>(sc, qf, sK, lane);
      softmax_tile<D / 8, TBN / 8>(sc, o, m, l, j0, row_lo, row_hi, scale_log2, lane);
      pv_tile<D, TBN / 8>(o, sc, sV, lane);
      __syncwarp();                // every lane is through with this stage
      issue(t + STAGES);
    }
  }
  cp_async_wait<0>();
  pdl_launch();                  // the stream's next kernel may start coming in now
  // The warps' partial results meet in shared memory (each warp's own stages are free by now) and leave the
  // CTA as one: rows < g, the running max, the sum and the unnormalised output, combined in warp order.
  {
    float* part = (float*)mine;                          // [g][D + 4]: output, max, sum, two unused (rows stay 16-byte aligned)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = (lane >> 2) + h * 8;
      if (r >= g) continue;
      float* dst = part + r * (D + 4) + (lane & 3) * 2;
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) *(float2*)(dst + nt * 8) = make_float2(o[nt][h * 2], o[nt][h * 2 + 1]);
      if ((lane & 3) == 0) { part[r * (D + 4) + D] = m[h]; part[r * (D + 4) + D + 1] = l[h]; }
    }
  }
  __syncthreads();
  for (int item = threadIdx.x; item < g * (D / 4); item += blockDim.x) {
    const int r = item / (D / 4), q4 = item - r * (D / 4);
    float mm = -INFINITY;
    for (int w = 0; w < nwarps; ++w)
      mm = fmaxf(mm, ((const float*)(smem_raw + (size_t)w * dec_warp_smem<D, STAGES, TBN>()))[r * (D + 4) + D]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float ll = 0.f;
    for (int w = 0; w < nwarps; ++w) {
      const float* pw = (const float*)(smem_raw + (size_t)w * dec_warp_smem<D, STAGES, TBN>()) + r * (D + 4);
      const float mw = pw[D];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      const float4 v = *(const float4*)(pw + q4 * 4);
      acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
      ll += pw[D + 1] * f;
    }
    const size_t slot = ((size_t)s * nq + kvh * g + r) * max_chunks + cta_x;
    *(float4*)(ws_o + slot * D + q4 * 4) = acc;
    if (q4 == 0) *(float2*)(ws_ml + slot * 2) = make_float2(mm, ll);
  }
  // the last CTA of this (sequence, kv head) merges the CTAs' results, in order
  // (the chunk size again from what it came from, rather than kept in a register through the tile loop)
  const int ck_m = (SMALL && (long long)gridDim.x * gridDim.y * ((len + CHUNK - 1) / CHUNK) < small_below) ? CHUNK_SMALL : CHUNK;
  const int ch_lo = kmin / ck_m, ch_hi = (len + ck_m - 1) / ck_m;
  const int cta_lo = ch_lo / nwarps, cta_hi = (ch_hi - 1) / nwarps + 1;
  const int ncta = cta_hi - cta_lo;
  __shared__ int s_last;
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(&counters[s * nkv + kvh], 1);
    s_last = (done == ncta - 1);
    if (s_last) counters[s * nkv + kvh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
  const int tid = threadIdx.x, nthr = blockDim.x;
  // Four outputs of a row and one half of its partial results a thread (neighbouring lanes hold the two
  // halves).  Eight results are fetched together (indices are clamped and the factor of one past the end is
  // 0, so that no load waits for a branch) and added under a running max, which is raised batch by batch;
  // then first half + second half.  The order depends on the sequence's own length only.
  const int half_n = (ncta + 1) >> 1;
  const int items = g * (D / 4) * 2;
  for (int it0 = 0; it0 < items; it0 += nthr) {
    const int item = it0 + tid;
    const bool valid = item < items;
    const int h = item & 1, q4 = (item >> 1) % (D / 4), r = valid ? (item >> 1) / (D / 4) : 0;
    const size_t base = ((size_t)s * nq + kvh * g + r) * max_chunks;
    const int c_begin = cta_lo + h * half_n, c_end = valid ? min(cta_hi, c_begin + half_n) : c_begin;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float ll = 0.f, mm = -INFINITY;
    for (int c0 = c_begin; c0 < c_end; c0 += 8) {
      float4 v[8];
      float2 ml[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = min(c0 + j, c_end - 1);
        v[j] = __ldcg((const float4*)(ws_o + (base + c) * D + q4 * 4));
        ml[j] = __ldcg((const float2*)(ws_ml + (base + c) * 2));
      }
      float bm = mm;
#pragma unroll
      for (int j = 0; j < 8; ++j) if (c0 + j < c_end) bm = fmaxf(bm, ml[j].x);
      if (bm == -INFINITY) continue;                       // nothing seen so far
      const float keep = mm == -INFINITY ? 0.f : exp2f(mm - bm);
      acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
      ll *= keep;
      mm = bm;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = (c0 + j < c_end && ml[j].x != -INFINITY) ? exp2f(ml[j].x - mm) : 0.f;
        ll += ml[j].y * f;
        acc.x += v[j].x * f; acc.y += v[j].y * f; acc.z += v[j].z * f; acc.w += v[j].w * f;
      }
    }
    // lane pairs (h = 0, 1) are neighbours: every lane of the warp takes part in the exchange
    float4 oth;
    oth.x = __shfl_xor_sync(0xffffffffu, acc.x, 1); oth.y = __shfl_xor_sync(0xffffffffu, acc.y, 1);
    oth.z = __shfl_xor_sync(0xffffffffu, acc.z, 1); oth.w = __shfl_xor_sync(0xffffffffu, acc.w, 1);
    const float llo = __shfl_xor_sync(0xffffffffu, ll, 1);
    const float mmo = __shfl_xor_sync(0xffffffffu, mm, 1);
    if (valid && h == 0) {
      const float top = fmaxf(mm, mmo);
      const float fa = mm == -INFINITY ? 0.f : exp2f(mm - top), fb = mmo == -INFINITY ? 0.f : exp2f(mmo - top);
      const float lt = ll * fa + llo * fb;
      const float inv = lt > 0.f ? 1.0f / lt : 0.f;
      bf16* o = out + ((size_t)s * nq + kvh * g + r) * D + q4 * 4;
      __nv_bfloat162 lo = __floats2bfloat162_rn((acc.x * fa + oth.x * fb) * inv, (acc.y * fa + oth.y * fb) * inv);
      __nv_bfloat162 hi = __floats2bfloat162_rn((acc.z * fa + oth.z * fb) * inv, (acc.w * fa + oth.w * fb) * inv);
      uint2 w;
      w.x = *(unsigned*)&lo; w.y = *(unsigned*)&hi;
      *(uint2*)o = w;
    }
  }
}

// ---------------------------------------------------------------------------
// entry points
// ---------------------------------------------------------------------------
static bool mma_supported(int nq, int nkv, int d) {
  if (nq <= 0 || nkv <= 0 || nq % nkv) return false;
  if (!(d == 16 || d == 32 || d == 64 || d == 128)) return false;
  return true;
}

template <int D> static size_t prefill_smem() { return (size_t)(BM + 4 * BN) * D * sizeof(bf16) + 2 * BN * sizeof(long long); }
template <int D>
static int launch_prefill(const bf16* q, int q_stride, bf16* out, const bf16* kc, const bf16* vc,
                          const int* bt, int max_blocks, const int* q_start, const int* seq_lens,
                          int seq_begin, int seq_end, int num_tokens, int nq, int nkv, int page_size,
                          int num_pages, int window, float scale, int* err, cudaStream_t stream) {
  const int g = nq / nkv;
  const int bq = BM / g;
  const int tiles = (num_tokens + bq - 1) / bq + (seq_end - seq_begin);
  const size_t smem = prefill_smem<D>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if ((long long)tiles * nkv > 0x7fffffffLL) return RLLM_E_UNSUPPORTED;
  dim3 grid(tiles * nkv);
  attention_prefill_kernel<D><<<grid, NTHREADS, smem, stream>>>(q, q_stride, out, kc, vc, bt, max_blocks, q_start,
      seq_lens, seq_begin, seq_end, nq, nkv, page_size, num_pages, window, scale * 1.4426950408889634f, err);
  RLLM_LAUNCH_CHECK();
  return 0;
}

// Prefill: sequences seq_begin .. seq_end-1 of the step, whose query tokens are
// rows q_start[s] .. q_start[s+1]-1 of q and out; num_tokens bounds their count.
RLLM_EXPORT int rllm_attention_prefill_bf16(const void* q, int q_stride, void* out, const void* kcache,
                                            const void* vcache, const int* block_table, int max_blocks,
                                            const int* q_start, const int* seq_lens, int seq_begin,
                                            int seq_end, int num_tokens, int nq, int nkv, int d, int page_size,
                                            int num_pages, int window, float scale, int* err,
                                            cudaStream_t stream) {
  if (seq_end <= seq_begin || num_tokens <= 0) return 0;
  if (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0 || q_stride % 8 || !(scale > 0.f))
    return RLLM_E_BADARG;
  if (!mma_supported(nq, nkv, d) || nq / nkv > BM) return RLLM_E_UNSUPPORTED;
#define RLLM_PREFILL(DD) return launch_prefill<DD>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)kcache, \
      (const bf16*)vcache, block_table, max_blocks, q_start, seq_lens, seq_begin, seq_end, num_tokens, nq, nkv, \
      page_size, num_pages, window, scale, err, stream)
  switch (d) {
    case 16: RLLM_PREFILL(16);
    case 32: RLLM_PREFILL(32);
    case 64: RLLM_PREFILL(64);
    case 128: RLLM_PREFILL(128);
  }
  return RLLM_E_UNSUPPORTED;
}

// floats of workspace that a decode call with these sizes needs
RLLM_EXPORT long long rllm_attention_decode_workspace(int num_seqs, int nq, int d, int max_seq_len) {
  const long long chunks = 2 * ((max_seq_len + CHUNK - 1) / CHUNK);     // (room for chunks of CHUNK_SMALL keys)
  return (long long)num_seqs * nq * chunks * (d + 2);
}

template <int D, int STAGES, int TBN, bool SMALL>
static int launch_decode_small(int warps, bf16* qkv, int q_stride, bf16* out, bf16* kc, bf16* vc, const int* bt,
                             int max_blocks, const int* seq_lens, int num_seqs, int nq, int nkv, int page_size,
                             int num_pages, int window, float scale, int max_chunks, const double* inv_freq,
                             int rotary_dim, int write_kv, float* ws, int* counters, int* err,
                             cudaStream_t stream, int small_below) {
  if (SMALL) max_chunks *= CHUNK / CHUNK_SMALL;      // the grid and the workspace's stride: room for the smaller chunks
  const size_t smem = (size_t)warps * dec_warp_smem<D, STAGES, TBN>();
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D, STAGES, TBN, SMALL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  float* ws_o = ws;
  float* ws_ml = ws + (size_t)num_seqs * nq * max_chunks * D;
  const unsigned per_seq = (unsigned)((max_chunks + warps - 1) / warps);
  dim3 grid = SMALL ? dim3(nkv, num_seqs, per_seq) : dim3(per_seq, nkv, num_seqs);
  static int resident[5];        // by number of warps
  if (!resident[warps]) resident[warps] = rllm_resident_ctas(attention_decode_kernel<D, STAGES, TBN, SMALL>, 32 * warps, smem) + 1;
  const long long ctas = (long long)grid.x * grid.y * grid.z;
  const int tail_from = (int)(ctas > resident[warps] - 1 ? ctas - (resident[warps] - 1) : 0);
  cudaError_t e = rllm_launch_pdl(attention_decode_kernel<D, STAGES, TBN, SMALL>, grid, dim3(32 * warps), smem, stream, qkv,
      q_stride, out, kc, vc, bt, max_blocks, seq_lens, nq, nkv, page_size, num_pages, window,
      scale * 1.4426950408889634f, max_chunks, inv_freq, rotary_dim, write_kv, ws_o, ws_ml, counters, err, tail_from,
      resident[warps] - 1, small_below);
  return (int)e;
}

template <int D, int STAGES, int TBN>
static int launch_decode_cfg(int warps, bf16* qkv, int q_stride, bf16* out, bf16* kc, bf16* vc, const int* bt,
                             int max_blocks, const int* seq_lens, int num_seqs, int nq, int nkv, int page_size,
                             int num_pages, int window, float scale, int max_chunks, const double* inv_freq,
                             int rotary_dim, int write_kv, float* ws, int* counters, int* err,
                             cudaStream_t stream, int small_below) {
#define RLLM_DEC_CFG_ARGS warps, qkv, q_stride, out, kc, vc, bt, max_blocks, seq_lens, num_seqs, nq, nkv, page_size, num_pages, \
      window, scale, max_chunks, inv_freq, rotary_dim, write_kv, ws, counters, err, stream, small_below
  if (small_below) return launch_decode_small<D, STAGES, TBN, true>(RLLM_DEC_CFG_ARGS);
  return launch_decode_small<D, STAGES, TBN, false>(RLLM_DEC_CFG_ARGS);
}

// Four warps a CTA.  With many chunks in all, one stage a warp, so that as many warps as possible are
// resident per SM and hide each other's loads (measured best at batch 8 and 64, for heads of 64 and of 128:
// 34.8 and 202 us at head size 128 against 49 and 298 us for two warps with three stages); with few chunks,
// two stages a warp (best at batch 1).  The choice changes no result.
template <int D>
static int launch_decode(bf16* qkv, int q_stride, bf16* out, bf16* kc, bf16* vc, const int* bt, int max_blocks,
                         const int* seq_lens, int num_seqs, int nq, int nkv, int page_size, int num_pages,
                         int window, float scale, int max_chunks, const double* inv_freq, int rotary_dim,
                         int write_kv, float* ws, int* counters, int* err, cudaStream_t stream, bool allow_small) {
  const long long total = (long long)max_chunks * nkv * num_seqs;
  // chunks of 64 keys are an option where even the longest sequences allowed would not make the work large
  // (the kernel decides sequence by sequence, by the sequence's own length)
  const int small_below = (allow_small && total < 4096) ? CHUNK_SMALL_BELOW : 0;
#define RLLM_DEC_ARGS qkv, q_stride, out, kc, vc, bt, max_blocks, seq_lens, num_seqs, nq, nkv, page_size, num_pages, \
      window, scale, max_chunks, inv_freq, rotary_dim, write_kv, ws, counters, err, stream, small_below
  // Heads of 128: a tile of 32 keys is 16 KB of K and V, and one stage a warp leaves the warp without loads
  // in flight while it multiplies; tiles of 16 keys in two stages keep them coming in the same shared memory
  // (batch 8 x 4,096 keys: 33.4 against 35.0 us; batch 32 x 2,096: 62.3 against 63.3 us; three CTAs an SM with
  // one stage of 16 keys and 168 registers: 41.2 and 61.6 us).
  if constexpr (D == 128) {
    if (total >= 1024) return launch_decode_cfg<D, 2, 16>(4, RLLM_DEC_ARGS);
  }
  if (total >= 1024) return launch_decode_cfg<D, 1, 32>(4, RLLM_DEC_ARGS);
  return launch_decode_cfg<D, 2, 32>(4, RLLM_DEC_ARGS);
}

// Decode: sequences 0 .. num_seqs-1 with one query token each.  Row s of qkv
// holds the token's q heads (and, with write_kv, its k and v heads behind them);
// row s of out receives the result.  rotary_dim > 0 rotates q (and k) here with
// the float64 frequency table inv_freq; write_kv stores the token's k and v into
// the cache.  max_seq_len bounds every seq_lens[s]; workspace holds
// rllm_attention_decode_workspace(...) floats; counters holds num_seqs * nkv
// ints that are zero before the call (the kernel leaves them zero).
// The kernel is launched with programmatic dependent launch.  With write_kv it reads seq_lens, the block
// table and the cache rows of earlier positions BEFORE it waits for the kernel ahead of it in the stream:
// these must be complete when that kernel starts, i.e. written by a kernel at least two launches ahead
// (or by a copy); only qkv may come from the kernel directly ahead.  Without write_kv it waits first.
// Every seq_lens[s] must be at least 1.
static int decode_bf16(void* qkv, int q_stride, void* out, void* kcache, void* vcache,
                       const int* block_table, int max_blocks, const int* seq_lens,
                       int num_seqs, int max_seq_len, int nq, int nkv, int d, int page_size,
                       int num_pages, int window, float scale, const double* inv_freq,
                       int rotary_dim, int write_kv, float* workspace, int* counters,
                       int* err, cudaStream_t stream, bool allow_small) {
  if (num_seqs <= 0) return 0;
  if (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0 || q_stride % 8 || max_seq_len <= 0 ||
      !workspace || !counters || !(scale > 0.f) || rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || (rotary_dim && !inv_freq))
    return RLLM_E_BADARG;
  if (!mma_supported(nq, nkv, d) || nq / nkv > 16) return RLLM_E_UNSUPPORTED;
  const int max_splits = (max_seq_len + CHUNK - 1) / CHUNK;
  if (max_splits > 65535 * 4 || num_seqs > 65535) return RLLM_E_UNSUPPORTED;
  if ((long long)num_pages * nkv * page_size > 0x7fffffffLL) return RLLM_E_UNSUPPORTED;   // cache rows are counted in an int
#define RLLM_DECODE(DD) return launch_decode<DD>((bf16*)qkv, q_stride, (bf16*)out, (bf16*)kcache, (bf16*)vcache, \
      block_table, max_blocks, seq_lens, num_seqs, nq, nkv, page_size, num_pages, window, scale, max_splits, \
      inv_freq, rotary_dim, write_kv, workspace, counters, err, stream, allow_small)
  switch (d) {
    case 16: RLLM_DECODE(16);
    case 32: RLLM_DECODE(32);
    case 64: RLLM_DECODE(64);
    case 128: RLLM_DECODE(128);
  }
  return RLLM_E_UNSUPPORTED;
}

RLLM_EXPORT int rllm_attention_decode_bf16(void* qkv, int q_stride, void* out, void* kcache, void* vcache,
                                           const int* block_table, int max_blocks, const int* seq_lens,
                                           int num_seqs, int max_seq_len, int nq, int nkv, int d, int page_size,
                                           int num_pages, int window, float scale, const double* inv_freq,
                                           int rotary_dim, int write_kv, float* workspace, int* counters,
                                           int* err, cudaStream_t stream) {
  return decode_bf16(qkv, q_stride, out, kcache, vcache, block_table, max_blocks, seq_lens, num_seqs, max_seq_len, nq,
                     nkv, d, page_size, num_pages, window, scale, inv_freq, rotary_dim, write_kv, workspace, counters,
                     err, stream, true);
}

// ---------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate: the scratch lives
// in this library's own device memory.  See attention_decode_static.h for who
// needs this and for the rules; nothing like it exists in the reference.
// ---------------------------------------------------------------------------
#include "attention_decode_static.h"
#include <atomic>

// partial results first, then the counters; fixed size, one per GPU that loads the library
static __device__ __align__(256) float rllm_decode_static_scratch[RLLM_DECODE_STATIC_FLOATS + RLLM_DECODE_STATIC_COUNTERS];

// Device address of the scratch array on the current device.  In host code the
// array's name is only a stand-in; a kernel must be given the address that
// cudaGetSymbolAddress reports.  Looked up once per device.
static int decode_static_address(float** ptr) {
  // Atomic so that two host threads may make their first call together: both look the address up (the
  // same value) and store it.
  static std::atomic<float*> cached[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return RLLM_E_UNSUPPORTED;
  float* p = cached[dev].load(std::memory_order_acquire);
  if (!p) {
    void* q = nullptr;
    e = cudaGetSymbolAddress(&q, rllm_decode_static_scratch);
    if (e != cudaSuccess) return (int)e;
    p = (float*)q;
    cached[dev].store(p, std::memory_order_release);
  }
  *ptr = p;
  return 0;
}

RLLM_EXPORT int rllm_attention_decode_bf16_static(void* qkv, int q_stride, void* out, void* kcache, void* vcache,
                                                  const int* block_table, int max_blocks, const int* seq_lens,
                                                  int num_seqs, int max_seq_len, int nq, int nkv, int d,
                                                  int page_size, int num_pages, int window, float scale,
                                                  const double* inv_freq, int rotary_dim, int write_kv, int* err,
                                                  cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || d <= 0 || max_seq_len <= 0) return RLLM_E_BADARG;
  // (the fixed array's limit counts chunks of CHUNK keys; the smaller chunks are an option while they fit too)
  const long long need = (long long)num_seqs * nq * ((max_seq_len + CHUNK - 1) / CHUNK) * (d + 2);
  const bool allow_small = rllm_attention_decode_workspace(num_seqs, nq, d, max_seq_len) <= RLLM_DECODE_STATIC_FLOATS;
  if (need > RLLM_DECODE_STATIC_FLOATS || (long long)num_seqs * nkv > RLLM_DECODE_STATIC_COUNTERS)
    return RLLM_E_STATIC_TOO_LARGE;
  float* scratch = nullptr;
  int rc = decode_static_address(&scratch);
  if (rc) return rc;
  int* counters = (int*)(scratch + RLLM_DECODE_STATIC_FLOATS);
  // the merge counters must start at zero; an earlier call that was cut short may have left them set
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)num_seqs * nkv * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  return decode_bf16(qkv, q_stride, out, kcache, vcache, block_table, max_blocks, seq_lens, num_seqs,
                     max_seq_len, nq, nkv, d, page_size, num_pages, window, scale, inv_freq,
                     rotary_dim, write_kv, scratch, counters, err, stream, allow_small);
}
