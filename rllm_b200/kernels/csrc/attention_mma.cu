// Paged causal attention for bfloat16 on tensor cores (mma.sync m16n8k16,
// float32 accumulate), grouped-query aware: the query heads that share a kv
// head are packed into the rows of one tile, so a K/V tile is loaded once for
// all of them.
//
//   prefill kernel  rows = (query token, head of the group); 4 warps x 16 rows;
//                   key tiles of 64, double-buffered with cp.async; online
//                   softmax in float32 (FlashAttention-2 schedule).
//   decode kernel   one query token per sequence; CTA = (256-key split, kv
//                   head, sequence); each of the 4 warps takes 64 keys of the
//                   split; partial (max, sum, output) go to a workspace and a
//                   combine kernel merges the splits in order.
//
// Contract as in attention_simt.cu: the query at position p of sequence s
// sees keys max(0, p - window + 1) .. p (window 0: all), read from the cache
// through the block table; kv head of head h is h / (nq / nkv); scores are
// scaled by `scale`; softmax and both accumulations are float32.  Key tiles and
// splits are aligned to absolute positions (multiples of 64 and 256), so a
// row's arithmetic does not depend on the batch around it or on how its
// sequence was cut into steps.
//
// The reference's kernels for the same job are one-thread-per-element CUDA-core
// loops (crates/rllm-kernels/src/cuda/paged_attention.cu:88-179, 252-347).
#include "common.cuh"
#include <math.h>

#define BM 64          // rows per CTA (prefill)
#define BN 64          // keys per tile
#define SPLIT 256      // keys per CTA (decode)
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

// Copy `rows` keys (positions j0 .. j0+rows-1 of the sequence) of one kv head
// from the paged cache into a tile; keys outside [lo, hi) are zero-filled.
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* tile, const bf16* __restrict__ cache,
                                             const int* __restrict__ bt, int j0, int rows, int lo, int hi,
                                             int kvh, int nkv, int page_size, int num_pages, int tid,
                                             int nthreads, int* err) {
  constexpr int C = D / 8;
  for (int idx = tid; idx < rows * C; idx += nthreads) {
    const int r = idx / C, c = idx - r * C;
    const int j = j0 + r;
    bool ok = j >= lo && j < hi;
    const bf16* src = cache;
    if (ok) {
      const int page = bt[j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, 4);
        ok = false;
      } else {
        src = cache + (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * D + c * 8;
      }
    }
    cp_async16(tile_ptr<D>(tile, r, c), src, ok);
  }
}

// S[16 x 64] = Q_frag . K_tile^T for one warp; accumulators s[8 n-tiles][4].
template <int D>
__device__ __forceinline__ void qk_tile(float (*s)[4], const unsigned (*qf)[4], bf16* sK, int lane) {
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < 4; ++np) {   // two n-tiles (16 keys) per ldmatrix.x4
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

// O[16 x D] += P[16 x 64] . V_tile for one warp; p given as accumulators.
template <int D>
__device__ __forceinline__ void pv_tile(float (*o)[4], const float (*p)[4], bf16* sV, int lane) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {     // 16 keys per k-step
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

// Online-softmax update of one warp's 16 x 64 score tile.  Thread holds rows
// r0 = lane/4 and r0 + 8; positions and key ranges per row are given.
//   s: raw scores in, probabilities out;  m, l: running max (log2 domain) and sum.
template <int DT>
__device__ __forceinline__ void softmax_tile(float (*s)[4], float (*o)[4], float* m, float* l, int j0,
                                             const int* row_lo, const int* row_hi, float scale_log2,
                                             int lane) {
  const int col0 = (lane & 3) * 2;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int hrow = e >> 1;
      const int j = j0 + nt * 8 + col0 + (e & 1);
      const bool vis = j >= row_lo[hrow] && j < row_hi[hrow];
      const float v = vis ? s[nt][e] * scale_log2 : -INFINITY;
      s[nt][e] = v;
      mx[hrow] = fmaxf(mx[hrow], v);
    }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
  }
  float corr[2], mnew[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mnew[h] = fmaxf(m[h], mx[h]);
    corr[h] = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - mnew[h]);
    if (mnew[h] == -INFINITY) corr[h] = 1.f;   // nothing seen yet: keep zeros
    m[h] = mnew[h];
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int hrow = e >> 1;
      const float p = (s[nt][e] == -INFINITY) ? 0.f : exp2f(s[nt][e] - mnew[hrow]);
      s[nt][e] = p;
      sum[hrow] += p;
    }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
    sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
    l[h] = l[h] * corr[h] + sum[h];
  }
#pragma unroll
  for (int nt = 0; nt < DT; ++nt) {
    o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
    o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
  }
}

// ---------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(NTHREADS)
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
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = nq / nkv;
  const int bq = BM / g;               // query tokens per tile (rows beyond bq * g stay idle)
  const int kvh = blockIdx.y;
  // which (sequence, tile) is this CTA?
  int s = -1, tile = 0;
  {
    int left = blockIdx.x;
    for (int i = seq_begin; i < seq_end; ++i) {
      const int n = (q_start[i + 1] - q_start[i] + bq - 1) / bq;
      if (left < n) { s = i; tile = left; break; }
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

  load_kv_tile<D>(sK, kcache, bt, tile_lo * BN, BN, kmin, kend, kvh, nkv, page_size, num_pages, tid, NTHREADS, err);
  load_kv_tile<D>(sV, vcache, bt, tile_lo * BN, BN, kmin, kend, kvh, nkv, page_size, num_pages, tid, NTHREADS, err);
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
    if (kt + 1 < tile_hi) {
      bf16* nK = sK + (stage ^ 1) * BN * D;
      bf16* nV = sV + (stage ^ 1) * BN * D;
      load_kv_tile<D>(nK, kcache, bt, (kt + 1) * BN, BN, kmin, kend, kvh, nkv, page_size, num_pages, tid, NTHREADS, err);
      load_kv_tile<D>(nV, vcache, bt, (kt + 1) * BN, BN, kmin, kend, kvh, nkv, page_size, num_pages, tid, NTHREADS, err);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float sc[8][4];
    qk_tile<D>(sc, qf, sK + stage * BN * D, lane);
    softmax_tile<D / 8>(sc, o, m, l, kt * BN, row_lo, row_hi, scale_log2, lane);
    pv_tile<D>(o, sc, sV + stage * BN * D, lane);
    __syncthreads();       // the next iteration overwrites the other stage, which is this one's successor
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
// decode: one query token per sequence, keys split over CTAs and warps
// workspace per (sequence, head, split): D floats of unnormalised output, then
// per (sequence, head, split) max (log2 domain) and sum.
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(NTHREADS)
attention_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kcache,
                        const bf16* __restrict__ vcache, const int* __restrict__ block_table,
                        int max_blocks, const int* __restrict__ seq_lens, int nq, int nkv, int page_size,
                        int num_pages, int window, float scale_log2, int max_splits,
                        float* __restrict__ ws_o, float* __restrict__ ws_ml, int* __restrict__ err) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  bf16* sQ = (bf16*)smem_raw;                        // [16][D]
  bf16* sK = sQ + 16 * D + warp * 2 * BN * D;        // this warp's [BN][D]
  bf16* sV = sK + BN * D;
  float* sO = (float*)(sQ + 16 * D + 4 * 2 * BN * D);   // [4 warps][16][D] partial outputs
  float* sML = sO + 4 * 16 * D;                          // [4][16][2]
  const int g = nq / nkv;
  const int split = blockIdx.x, kvh = blockIdx.y, s = blockIdx.z;
  const int len = seq_lens[s];
  const int pos = len - 1;
  const int kmin = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int c0 = split * SPLIT;
  if (c0 >= len || c0 + SPLIT <= kmin) return;      // this split holds no visible key
  const int* bt = block_table + (size_t)s * max_blocks;

  // Q rows = heads of the group, rows >= g zero
  {
    constexpr int C = D / 8;
    for (int idx = tid; idx < 16 * C; idx += NTHREADS) {
      const int r = idx / C, c = idx - r * C;
      const bool ok = r < g;
      const bf16* src = ok ? q + (size_t)s * q_stride + (size_t)(kvh * g + r) * D + c * 8 : q;
      cp_async16(tile_ptr<D>(sQ, r, c), src, ok);
    }
  }
  const int j0 = c0 + warp * BN;
  const bool active = j0 < len && j0 + BN > kmin;
  if (active) {
    load_kv_tile<D>(sK, kcache, bt, j0, BN, kmin, len, kvh, nkv, page_size, num_pages, lane, 32, err);
  }
  cp_async_commit();
  if (active) {
    load_kv_tile<D>(sV, vcache, bt, j0, BN, kmin, len, kvh, nkv, page_size, num_pages, lane, 32, err);
  }
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();                                   // Q (all threads) and this warp's K are in

  float o[D / 8][4];
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  if (active) {
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
    float sc[8][4];
    qk_tile<D>(sc, qf, sK, lane);
    softmax_tile<D / 8>(sc, o, m, l, j0, row_lo, row_hi, scale_log2, lane);
    cp_async_wait<0>();
    __syncwarp();
    pv_tile<D>(o, sc, sV, lane);
  } else {
    cp_async_wait<0>();
  }
  // hand the warp's partial to shared memory
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + h * 8;
    float* dst = sO + ((size_t)warp * 16 + r) * D + (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      dst[nt * 8] = o[nt][h * 2];
      dst[nt * 8 + 1] = o[nt][h * 2 + 1];
    }
    if ((lane & 3) == 0) {
      sML[(warp * 16 + r) * 2] = m[h];
      sML[(warp * 16 + r) * 2 + 1] = l[h];
    }
  }
  __syncthreads();
  // merge the four warps in order and write this split's partial
  for (int idx = tid; idx < g * D; idx += NTHREADS) {
    const int r = idx / D, dcol = idx - r * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sML[(w * 16 + r) * 2]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sML[(w * 16 + r) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      acc += sO[((size_t)w * 16 + r) * D + dcol] * f;
      ll += sML[(w * 16 + r) * 2 + 1] * f;
    }
    const size_t slot = ((size_t)s * nq + kvh * g + r) * max_splits + split;
    ws_o[slot * D + dcol] = acc;
    if (dcol == 0) { ws_ml[slot * 2] = mm; ws_ml[slot * 2 + 1] = ll; }
  }
}

// out[s, h, :] = sum over the sequence's splits, in order, rescaled to the common max
template <int D>
__global__ void attention_combine_kernel(bf16* __restrict__ out, const float* __restrict__ ws_o,
                                         const float* __restrict__ ws_ml, const int* __restrict__ seq_lens,
                                         int nq, int window, int max_splits) {
  const int h = blockIdx.x, s = blockIdx.y;
  const int len = seq_lens[s];
  const int pos = len - 1;
  const int kmin = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int sp_lo = kmin / SPLIT, sp_hi = (len + SPLIT - 1) / SPLIT;
  const size_t base = ((size_t)s * nq + h) * max_splits;
  float mm = -INFINITY;
  for (int sp = sp_lo; sp < sp_hi; ++sp) mm = fmaxf(mm, ws_ml[(base + sp) * 2]);
  for (int dcol = threadIdx.x; dcol < D; dcol += blockDim.x) {
    float acc = 0.f, ll = 0.f;
    for (int sp = sp_lo; sp < sp_hi; ++sp) {
      const float mw = ws_ml[(base + sp) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      acc += ws_o[(base + sp) * D + dcol] * f;
      ll += ws_ml[(base + sp) * 2 + 1] * f;
    }
    out[((size_t)s * nq + h) * D + dcol] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
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

template <int D> static size_t prefill_smem() { return (size_t)(BM + 4 * BN) * D * sizeof(bf16); }
template <int D> static size_t decode_smem() {
  return (size_t)(16 + 8 * BN) * D * sizeof(bf16) + (size_t)4 * 16 * D * sizeof(float) + 4 * 16 * 2 * sizeof(float);
}

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
  dim3 grid(tiles, nkv);
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
  if (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0 || q_stride % 8) return RLLM_E_BADARG;
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
  const long long splits = (max_seq_len + SPLIT - 1) / SPLIT;
  return (long long)num_seqs * nq * splits * (d + 2);
}

template <int D>
static int launch_decode(const bf16* q, int q_stride, bf16* out, const bf16* kc, const bf16* vc, const int* bt,
                         int max_blocks, const int* seq_lens, int num_seqs, int nq, int nkv, int page_size,
                         int num_pages, int window, float scale, int max_splits, float* ws, int* err,
                         cudaStream_t stream) {
  const size_t smem = decode_smem<D>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  float* ws_o = ws;
  float* ws_ml = ws + (size_t)num_seqs * nq * max_splits * D;
  dim3 grid(max_splits, nkv, num_seqs);
  attention_decode_kernel<D><<<grid, NTHREADS, smem, stream>>>(q, q_stride, kc, vc, bt, max_blocks, seq_lens, nq, nkv,
      page_size, num_pages, window, scale * 1.4426950408889634f, max_splits, ws_o, ws_ml, err);
  RLLM_LAUNCH_CHECK();
  dim3 cgrid(nq, num_seqs);
  attention_combine_kernel<D><<<cgrid, D < 32 ? 32 : D, 0, stream>>>(out, ws_o, ws_ml, seq_lens, nq, window, max_splits);
  RLLM_LAUNCH_CHECK();
  return 0;
}

// Decode: sequences 0 .. num_seqs-1 with one query token each (row s of q and
// out).  max_seq_len bounds every seq_lens[s]; workspace holds
// rllm_attention_decode_workspace(...) floats.
RLLM_EXPORT int rllm_attention_decode_bf16(const void* q, int q_stride, void* out, const void* kcache,
                                           const void* vcache, const int* block_table, int max_blocks,
                                           const int* seq_lens, int num_seqs, int max_seq_len, int nq, int nkv,
                                           int d, int page_size, int num_pages, int window, float scale,
                                           float* workspace, int* err, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0 || q_stride % 8 || max_seq_len <= 0 ||
      !workspace)
    return RLLM_E_BADARG;
  if (!mma_supported(nq, nkv, d) || nq / nkv > 16) return RLLM_E_UNSUPPORTED;
  const int max_splits = (max_seq_len + SPLIT - 1) / SPLIT;
  if (max_splits > 65535 || num_seqs > 65535) return RLLM_E_UNSUPPORTED;
#define RLLM_DECODE(DD) return launch_decode<DD>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)kcache, \
      (const bf16*)vcache, block_table, max_blocks, seq_lens, num_seqs, nq, nkv, page_size, num_pages, window, \
      scale, max_splits, workspace, err, stream)
  switch (d) {
    case 16: RLLM_DECODE(16);
    case 32: RLLM_DECODE(32);
    case 64: RLLM_DECODE(64);
    case 128: RLLM_DECODE(128);
  }
  return RLLM_E_UNSUPPORTED;
}
