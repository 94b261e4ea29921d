// Paged causal attention over prompt portions for bfloat16 on the tcgen05
// tensor cores (head sizes 64 and 128): both products of attention, S = Q K^T
// and P V, run as tcgen05.mma with accumulators in tensor memory.
//
// One CTA per (tile of 128 rows, kv head, sequence); a row is a (query token,
// head of the kv head's group) pair, so 128 / g tokens share every K/V tile
// (if g does not divide 128 the last rows of a tile stay unused).
// Key tiles hold BN = 8192 / D keys (128 for head size 64, 64 for 128), so that a
// K or V stage is 16 KB either way, and two CTAs share an SM (their tensor memory too:
// 256 columns each).
// Q, K and V lie in shared memory as panels of 64 columns (128 bytes, the span of the
// 128-byte swizzle) by head dims; the probabilities P go from the softmax warps'
// registers into tensor memory (two bfloat16 a column) and are the A operand of
// P V from there: no shared memory, no fence between the proxies.
//   warp 0     TMA producer: Q once (3-D boxes: 64 dims x g heads x 128/g tokens),
//              then per tile the K and V rows of its cache pages (one 2-D box per
//              page and panel), into two-stage rings of their own; pages a sequence
//              does not hold are skipped.
//   warp 1     allocates TMEM (S: BN columns, output: D, P: BN / 2) and issues the
//              MMAs: S = Q K^T (128 x BN x D, both operands K-major), then, when
//              the softmax warps have left P in tensor memory, output += P V
//              (128 x D x BN; V is the MN-major operand, straight from its cache
//              layout).
//   warps 2-9  softmax, two threads a row (= TMEM lane): read the row's scores
//              with tcgen05.ld, mask (causal, window), keep a reference max and the
//              sum in float32, write P as bfloat16 pairs with tcgen05.st; the
//              output stays in TMEM and is rescaled only when a row's max has grown
//              by more than 2^8.  The two threads of a row swap their maxima
//              through spare columns behind P (heads of 128) or through columns
//              of S that each has already read (heads of 64: no column is spare).
// Contract and tile alignment as in attention_mma.cu (key tiles at absolute
// positions; a row's arithmetic does not depend on the batch).
// Every mbarrier wait is bounded (bit 16 of the error word, then wind-down).
// No cluster, no multicast.
#include "tcgen05.cuh"
#include <math.h>

#ifndef AT_POLY
// With heads of 64 the special-function unit bounds the kernel (1,024 cycles of ex2 a tile against 512 of MMA):
// one group of four exponentials in AT_POLY is computed on the FMA pipe instead (0: none).  Measured at
// 8,192 tokens: none 404 us, a quarter 373 us, a third 377 us, half 417 us.
#define AT_POLY 4
#endif
#define AT_BM 128
#define AT_THREADS 320
#define AT_STAGE 16384          // bytes of a K or V stage: BN keys x D dims

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, void* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(tg_smem(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(z), "r"(tg_smem(bar)) : "memory");
}
__device__ __forceinline__ float at_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The softmax warps' arithmetic uses the instructions of sm_100 that do two float32 operations
// (fma.rn.f32x2, add.rn.f32x2 on register pairs) or take three inputs (max.f32): a quarter fewer
// instructions a tile (measured: 2 to 3 % less time at 8,192 tokens; the exponentials and the
// hand-overs between warps weigh more).
__device__ __forceinline__ float at_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ unsigned long long at_pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void at_unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long at_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long at_add2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for two numbers at once without the special-function unit: x = n + f with n whole and |f| <= 1/2 (the
// 1.5 * 2^23 trick), a polynomial of degree 4 for 2^f (relative error 4e-5, far below bfloat16's step), and n
// added into the exponent bits.  x below -126 gives 2^-126 (as good as 0 beside a sum that is at least 2^-8).
__device__ __forceinline__ void at_exp2_poly2(unsigned long long x2, float& r0, float& r1) {
  float x0, x1;
  at_unpack2(x2, x0, x1);
  x2 = at_pack2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
  const unsigned long long magic = at_pack2(12582912.0f, 12582912.0f), nmagic = at_pack2(-12582912.0f, -12582912.0f);
  const unsigned long long t2 = at_add2(x2, magic);
  const unsigned long long n2 = at_add2(t2, nmagic);
  const unsigned long long f2 = at_fma2(n2, at_pack2(-1.0f, -1.0f), x2);
  unsigned long long p2 = at_fma2(at_pack2(0.0096181291f, 0.0096181291f), f2, at_pack2(0.0555041087f, 0.0555041087f));
  p2 = at_fma2(p2, f2, at_pack2(0.2402265070f, 0.2402265070f));
  p2 = at_fma2(p2, f2, at_pack2(0.6931471806f, 0.6931471806f));
  p2 = at_fma2(p2, f2, at_pack2(1.0f, 1.0f));
  float p0, p1, t0, t1;
  at_unpack2(p2, p0, p1);
  at_unpack2(t2, t0, t1);
  r0 = __uint_as_float(__float_as_uint(p0) + (__float_as_uint(t0) << 23));
  r1 = __uint_as_float(__float_as_uint(p1) + (__float_as_uint(t1) << 23));
}

// Two CTAs fit one SM, so that one CTA's softmax runs beside the other's products.
// The two threads of a row (one in warp w, one in warp w + 4, same TMEM lane) swap one value:
// each stores its own into a column of its own (`t_mine`, among the score columns it has read) and
// reads the other's (`t_theirs`) after the pair's mbarrier (two arrivals, one a warp; exchange n
// completes phase n).  Exchanges take two columns in turn: a column is used again two exchanges
// later at the earliest, when the partner, having passed the barrier between, has read it.  The
// columns may be score columns that the thread has read: the next tile's scores are written over
// them only after both have told the MMA warp that they are through with the tile.  False if the
// wait ran out.
__device__ __forceinline__ bool pair_exchange(unsigned t_mine, unsigned t_theirs, void* bar, int n, float mine, float* theirs, int* err) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(t_mine), "r"(__float_as_uint(mine)) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
  if (!__all_sync(0xffffffffu, mbar_wait(bar, n & 1, err))) return false;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  unsigned other;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(other) : "r"(t_theirs) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  *theirs = __uint_as_float(other);
  return true;
}

// Q, two stages of K and of V, barriers: two CTAs fit one SM
template <int AT_D> constexpr int at_smem_bytes() { return (AT_D / 64) * 16384 + 2 * AT_STAGE + 2 * AT_STAGE + 512; }

template <int AT_D>
__global__ void __launch_bounds__(AT_THREADS, 2)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ q_start,
                         const int* __restrict__ seq_lens, int seq_begin, int seq_end, int nq, int nkv,
                         int page_size, int num_pages, int window, float scale_log2, int* __restrict__ err) {
  constexpr int AT_BN = 8192 / AT_D;              // keys a tile
  constexpr int DP = AT_D / 64;                   // panels of head dims (Q, K, V)
  constexpr int KPANEL = AT_BN * 128;             // bytes of a K or V panel: BN rows of 128 bytes
  extern __shared__ __align__(1024) unsigned char at_raw[];
  unsigned char* base = at_raw;
  if (tg_smem(base) & 1023u) {                    // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicOr(err, 32);
    return;
  }
  unsigned char* sQ = base;                       // DP panels x [128 rows][64 dims] bf16, 128B swizzle
  unsigned char* sK = sQ + DP * 16384;            // 2 stages x DP panels x [BN keys][64 dims]
  unsigned char* sV = sK + 2 * AT_STAGE;          // 2 stages x DP panels x [BN keys][64 dims]
  unsigned long long* bars = (unsigned long long*)(sV + 2 * AT_STAGE);
  unsigned long long* q_full = bars;              // TMA -> MMA
  unsigned long long* k_full = bars + 1;          // [2] TMA -> MMA
  unsigned long long* k_empty = bars + 3;         // [2] MMA -> TMA: the scores that read the stage are done
  unsigned long long* v_full = bars + 5;          // [2] TMA -> MMA (and the softmax warps, for the last tile)
  unsigned long long* v_empty = bars + 7;         // [2] MMA -> TMA: the product that read the stage is done
  unsigned long long* s_full = bars + 9;          // MMA -> softmax
  unsigned long long* p_full = bars + 10;         // softmax (8 warps) -> MMA
  unsigned long long* pv_full = bars + 11;        // MMA -> softmax
  unsigned long long* s_free = bars + 12;         // softmax (8 warps) -> MMA
  unsigned long long* xbar = bars + 13;           // [4] the two warps of a row quarter, one another
  unsigned* tmem_slot = (unsigned*)(bars + 17);
  int* s_pages = (int*)(bars + 18);               // [4 tiles][8 boxes]: the producer's page numbers, from K's request to V's
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = nq / nkv;
  const int bq = AT_BM / g;                        // query tokens per tile
  const int kvh = blockIdx.x % nkv;
  // which (sequence, tile): the tiles that see the most keys get the lowest block indices, for every kv head
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
  const int pos0 = seq_lens[s] - qlen;
  const int t0 = tile * bq;
  const int ntok = min(bq, qlen - t0);
  const int first_pos = pos0 + t0, last_pos = pos0 + t0 + ntok - 1;
  const int kmin = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
  const int kend = last_pos + 1;
  const int tile_lo = kmin / AT_BN, tile_hi = (kend + AT_BN - 1) / AT_BN;
  const int* bt = block_table + (size_t)s * max_blocks;

  // stale rows of K and V (pages that are skipped) must hold finite numbers: clear the ring once
  for (int i = threadIdx.x; i < 4 * AT_STAGE / 16; i += AT_THREADS) ((uint4*)sK)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);
    mbar_init(pv_full, 1);
    mbar_init(s_free, 8);
    for (int i = 0; i < 4; ++i) mbar_init(&xbar[i], 2);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tg_smem(tmem_slot)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the cleared ring, before TMA writes into it
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_s = *tmem_slot, tmem_o = tmem_s + AT_BN, tmem_p = tmem_o + AT_D;   // BN + D + BN / 2 <= 256 columns

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, (unsigned)(DP * bq * g * 128));     // bq * g rows of the 128 (all of them if g divides 128)
      for (int dp = 0; dp < DP; ++dp) tma_load_3d(sQ + dp * 16384, &map_q, dp * 64, kvh * g, qs + t0, q_full);
    }
    // Lanes 0-7 fetch the boxes of a tile (a page and a panel of 64 dims each).  K and V have rings of their own: a K stage is
    // free once the scores that read it are done, a V stage once its product is, so K runs a tile further
    // ahead.  Lane 0 polls both rings.  (A request costs the warp about 140 cycles, eight boxes 1,100: with
    // pages of 16 keys the requests, not the bytes, bound how fast tiles come in.)
    const int boxes = (AT_BN / page_size) * DP;     // page_size divides BN; at most 8 boxes
    const int bpage = lane / DP, bpanel = lane % DP; // this lane's box: which page of the tile, which panel
    const int ntiles = tile_hi - tile_lo;
    // The page of this lane's box in tile `it`: read from the block table a tile ahead of its use (the load
    // is on its way while the warp polls), checked when the tile's keys are asked for, and kept in shared
    // memory until the tile's values are asked for (K runs at most three tiles ahead of V).
    auto fetch = [&](int it) {
      const int j = (tile_lo + it) * AT_BN + bpage * page_size;
      return (lane < boxes && it < ntiles && j < kend) ? bt[j / page_size] : -2;      // -2: no box
    };
    auto checked = [&](int it, int raw) {
      if (raw == -2) return -1;
      if (raw < 0 || raw >= num_pages) {
        const int j = (tile_lo + it) * AT_BN + bpage * page_size;
        if (j + page_size > kmin && bpanel == 0) atomicOr(err, 4);   // a page with visible keys is missing
        return -1;
      }
      return raw;
    };
    auto issue = [&](unsigned char* ring, const CUtensorMap* map, unsigned long long* full, int it, int page) {
      const int st = it & 1;
      const unsigned have = __ballot_sync(0xffffffffu, page >= 0);
      if (lane == 0) mbar_expect_tx(&full[st], (unsigned)(__popc(have) * page_size * 128));
      __syncwarp();
      if (page >= 0)
        tma_load_2d(ring + st * AT_STAGE + bpanel * KPANEL + bpage * page_size * 128, map, bpanel * 64,
                    (page * nkv + kvh) * page_size, &full[st]);
    };
    int nk = 0, nv = 0;                              // tiles whose K, V have been asked for
    int raw_next = fetch(0);
    unsigned spin = 0;
    while (nk < ntiles || nv < ntiles) {
      unsigned ready = 0;
      if (lane == 0) {
        if (nk < ntiles && nk - nv < 4 && mbar_test(&k_empty[nk & 1], ((nk >> 1) & 1) ^ 1)) ready |= 1u;
        if (nv < nk && mbar_test(&v_empty[nv & 1], ((nv >> 1) & 1) ^ 1)) ready |= 2u;
      }
      ready = __shfl_sync(0xffffffffu, ready, 0);
      if (!ready) {
        if (++spin > TG_SPIN_LIMIT) { if (lane == 0) atomicOr(err, 16); break; }
        continue;
      }
      spin = 0;
      if (ready & 1u) {
        const int page = checked(nk, raw_next);
        if (lane < 8) s_pages[(nk & 3) * 8 + lane] = page;
        raw_next = fetch(nk + 1);
        issue(sK, &map_k, k_full, nk, page);
        ++nk;
      }
      if (ready & 2u) {
        issue(sV, &map_v, v_full, nv, lane < 8 ? s_pages[(nv & 3) * 8 + lane] : -1);
        ++nv;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // S: float32 accumulate, bf16 x bf16, A and B K-major, M 128, N BN.
      // PV: the same with N = D, A (P) in tensor memory and B (V) MN-major.
      const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(AT_BN >> 3) << 17) | ((unsigned)(AT_BM >> 4) << 24);
      // (all D dims in one instruction: for D = 128 the two panels of V are a leading-dimension step apart)
      const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(AT_D >> 3) << 17) | ((unsigned)(AT_BM >> 4) << 24);
      const int ntiles = tile_hi - tile_lo;
      const unsigned long long dq = umma_desc(sQ);
      // scores of the tile in stage st: D / 16 steps along the head dims, panel by panel
      auto scores = [&](int st) {
        const unsigned long long dk = umma_desc(sK + st * AT_STAGE);
#pragma unroll
        for (int k = 0; k < AT_D / 16; ++k) {
          const unsigned long long a = dq + (unsigned long long)((k >> 2) * (16384 >> 4) + 2 * (k & 3));
          const unsigned long long b = dk + (unsigned long long)((k >> 2) * (KPANEL >> 4) + 2 * (k & 3));
          umma_bf16(tmem_s, a, b, idesc_s, k != 0);
        }
      };
      bool ok = mbar_wait(q_full, 0, err) && mbar_wait(&k_full[0], 0, err);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        scores(0);
        umma_commit(s_full);
        umma_commit(&k_empty[0]);
      }
      for (int it = 0; it < ntiles && ok; ++it) {
        const int st = it & 1;
        if (it + 1 < ntiles) {
          // the next tile's scores, as soon as its keys are here and the softmax warps hold this tile's scores
          const int sn = (it + 1) & 1;
          ok = mbar_wait(&k_full[sn], ((it + 1) >> 1) & 1, err) && mbar_wait(s_free, it & 1, err);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          scores(sn);
          umma_commit(s_full);
          umma_commit(&k_empty[sn]);
        }
        ok = mbar_wait(&v_full[st], (it >> 1) & 1, err) && mbar_wait(p_full, it & 1, err);   // P is in tensor memory, O is rescaled
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // V is the MN-major operand: 64 dims x 8 keys a swizzle atom, 8 keys on 1024 bytes further (stride
        // field), 64 dims on a panel further (leading-dimension field)
        const unsigned long long dv = (umma_desc(sV + st * AT_STAGE) & ~(0x3FFFull << 16)) | ((unsigned long long)(KPANEL >> 4) << 16);
#pragma unroll
        for (int kk = 0; kk < AT_BN / 16; ++kk)         // 16 keys a step: 8 columns of P on, V two row groups on
          umma_bf16_tmem_a(tmem_o, tmem_p + kk * 8, dv + (unsigned long long)(kk * (2048 >> 4)), idesc_pv,
                           (it != 0) || (kk != 0));
        umma_commit(pv_full);
        umma_commit(&v_empty[st]);
      }
    }
    __syncwarp();
  } else {
    // Two threads a row: warps 2-5 take the first half of the tile's keys (and of the output dims),
    // warps 6-9 the second; warp w and warp w + 4 own the same 32 rows (TMEM lanes) and exchange
    // the row's max and sum through score columns that they have read, under a barrier of their own.
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;               // this thread's row of the tile
    const int tl = r / g, hl = r - tl * g;
    const bool live = tl < ntok;
    // rows behind the portion's last token compute like the others; their result is not stored
    const int pos = pos0 + t0 + tl;
    const int row_hi = pos + 1;
    const int row_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    // tiles all of whose keys every row sees need no mask
    const int clear_lo = (window > 0 && pos0 + t0 + bq - window > 0) ? pos0 + t0 + bq - window : 0;
    const int clear_hi = first_pos + 1;
    float m_ref = -INFINITY, l = 0.f;
    const unsigned lane_sel = (unsigned)(quarter * 32) << 16;
    const int ntiles = tile_hi - tile_lo;
    constexpr int HC = AT_BN / 2;                    // keys a thread
    // Where the two threads of a row swap values: in spare columns behind P if the CTA's 256 columns leave
    // four (heads of 128); else in the score columns that each thread has read itself (its first two), and
    // then the MMA warp may write the next tile's scores only when the exchange is over.
    constexpr bool X_SPARE = AT_BN + AT_D + AT_BN / 2 + 4 <= 256;
    const unsigned x_mine = X_SPARE ? tmem_p + AT_BN / 2 + lane_sel + half * 2 : tmem_s + lane_sel + half * HC;
    const unsigned x_theirs = X_SPARE ? tmem_p + AT_BN / 2 + lane_sel + (half ^ 1) * 2 : tmem_s + lane_sel + (half ^ 1) * HC;
    bool ok = true;
    for (int it = 0; it < ntiles; ++it) {
      const int j0 = (tile_lo + it) * AT_BN;
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, it & 1, err));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float sc[HC];
#pragma unroll
      for (int c0 = 0; c0 < HC; c0 += 32) tmem_ld32(tmem_s + lane_sel + half * HC + c0, (unsigned*)(sc + c0));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (X_SPARE) {                                   // the scores are in registers: the next tile's may come
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
      }
      if (!(j0 >= clear_lo && j0 + AT_BN <= clear_hi)) {
        const unsigned lo_rel = (unsigned)(row_lo - j0 - half * HC), span = (unsigned)(row_hi - row_lo);
#pragma unroll
        for (int j = 0; j < HC; ++j)
          if (!((unsigned)j - lo_rel < span)) sc[j] = -INFINITY;
      }
      float mx0 = fmaxf(sc[0], sc[1]), mx1 = fmaxf(sc[2], sc[3]), mx2 = fmaxf(sc[4], sc[5]), mx3 = fmaxf(sc[6], sc[7]);
#pragma unroll
      for (int j = 8; j < HC; j += 8) {
        mx0 = at_max3(mx0, sc[j], sc[j + 1]); mx1 = at_max3(mx1, sc[j + 2], sc[j + 3]);
        mx2 = at_max3(mx2, sc[j + 4], sc[j + 5]); mx3 = at_max3(mx3, sc[j + 6], sc[j + 7]);
      }
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      float mx_other;
      ok = pair_exchange(x_mine + (it & 1), x_theirs + (it & 1), &xbar[quarter], it, mx, &mx_other, err);
      if (!ok) break;
      if (!X_SPARE) {                                  // through with the tile's score columns, the exchange's too
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
      }
      mx = fmaxf(mx, mx_other) * scale_log2;
      // The reference point of the exponentials moves only when the max has grown by more than 2^8: until
      // then the old one serves (probabilities up to 256, the sum and the output scale alike), and the
      // output accumulated so far needs no rescaling.  The rule looks at this row's scores only.
      const bool moves = mx > m_ref + 8.0f;
      float corr = 1.0f;
      if (moves) {
        corr = at_ex2(m_ref - mx);                    // from -inf: 0, and nothing has been summed yet
        m_ref = mx;
        l *= corr;
      }
      const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
      unsigned pk[HC / 2];
      const unsigned long long scale2 = at_pack2(scale_log2, scale_log2), shift2 = at_pack2(-m_safe, -m_safe);
      unsigned long long sum01 = at_pack2(0.f, 0.f), sum23 = sum01;
#pragma unroll
      for (int j = 0; j < HC; j += 4) {
        float p0, p1, p2, p3;
        if (AT_POLY > 0 && AT_D == 64 && (j / 4) % AT_POLY == AT_POLY - 1) {
          at_exp2_poly2(at_fma2(at_pack2(sc[j], sc[j + 1]), scale2, shift2), p0, p1);
          at_exp2_poly2(at_fma2(at_pack2(sc[j + 2], sc[j + 3]), scale2, shift2), p2, p3);
        } else {
          float x0, x1, x2, x3;
          at_unpack2(at_fma2(at_pack2(sc[j], sc[j + 1]), scale2, shift2), x0, x1);
          at_unpack2(at_fma2(at_pack2(sc[j + 2], sc[j + 3]), scale2, shift2), x2, x3);
          p0 = at_ex2(x0); p1 = at_ex2(x1); p2 = at_ex2(x2); p3 = at_ex2(x3);
        }
        sum01 = at_add2(sum01, at_pack2(p0, p1));
        sum23 = at_add2(sum23, at_pack2(p2, p3));
        __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
        pk[j / 2] = *(unsigned*)&h0;
        pk[j / 2 + 1] = *(unsigned*)&h1;
      }
      {
        float sum0, sum1, sum2, sum3;
        at_unpack2(sum01, sum0, sum1);
        at_unpack2(sum23, sum2, sum3);
        l += (sum0 + sum1) + (sum2 + sum3);
      }
      // the product of the tile before has to be through: it read P, and it wrote the output that is rescaled here
      if (it > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(pv_full, (it - 1) & 1, err));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (__any_sync(0xffffffffu, moves)) {
#pragma unroll
          for (int c0 = 0; c0 < AT_D / 2; c0 += 32) {
            unsigned v[32];
            tmem_ld32(tmem_o + lane_sel + half * (AT_D / 2) + c0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
            tmem_st32(tmem_o + lane_sel + half * (AT_D / 2) + c0, v);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      // this thread's keys half * HC .. + HC - 1: columns half * HC / 2 .. of P, two keys a column
      if constexpr (HC == 64) tmem_st32(tmem_p + lane_sel + half * (HC / 2), pk);
      else tmem_st16(tmem_p + lane_sel + half * (HC / 2), pk);
      // rows of V at and behind the last visible key were never written by this sequence: whatever
      // they hold must not reach the product (0 x inf), so they are cleared before P V is issued
      if (it == ntiles - 1) {
        ok = __all_sync(0xffffffffu, mbar_wait(&v_full[it & 1], (it >> 1) & 1, err));   // V has landed: nothing overwrites the zeros
        if (!ok) break;
      }
      if (it == ntiles - 1) {
        if (r < AT_BN && j0 + r >= kend) {            // thread r: key row r, half a row of every panel
#pragma unroll
          for (int dp = 0; dp < DP; ++dp) {
            uint4* vrow = (uint4*)(sV + (it & 1) * AT_STAGE + dp * KPANEL + r * 128 + half * 64);
#pragma unroll
            for (int c = 0; c < 4; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeros, before the MMA reads V
      }
      // hand P to the MMA warp
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(pv_full, (ntiles - 1) & 1, err));
    // the row's sum is the two halves' sums (an exchange slot no tile is using: the pair's last
    // exchange was for tile ntiles-1, this one takes the other parity)
    float lother = 0.f;
    if (ok) ok = pair_exchange(x_mine + (ntiles & 1), x_theirs + (ntiles & 1), &xbar[quarter], ntiles, l, &lother, err);
    const float lsum = half == 0 ? l + lother : lother + l;
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
      bf16* orow = out + ((size_t)(qs + t0 + tl) * nq + kvh * g + hl) * AT_D + half * (AT_D / 2);
#pragma unroll
      for (int c0 = 0; c0 < AT_D / 2; c0 += 32) {
        unsigned v[32];
        tmem_ld32(tmem_o + lane_sel + half * (AT_D / 2) + c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (live) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 w;
            __nv_bfloat162* h = (__nv_bfloat162*)&w;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              h[q] = __floats2bfloat162_rn(__uint_as_float(v[c + 2 * q]) * inv, __uint_as_float(v[c + 2 * q + 1]) * inv);
            *(uint4*)(orow + c0 + c) = w;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(256) : "memory");
  }
}

// ---------------------------------------------------------------------------
static int at_encode(CUtensorMap* map, int rank, const void* ptr, const cuuint64_t* dims, const cuuint64_t* strides,
                     const cuuint32_t* box) {
  tg_encode_fn enc = tg_get_encode();
  if (!enc) return RLLM_E_UNSUPPORTED;
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : RLLM_E_BADARG;
}

template <int D>
static int at_launch(const void* q, int q_stride, int num_q_rows, void* out, const void* kcache, const void* vcache,
                     const int* block_table, int max_blocks, const int* q_start, const int* seq_lens, int seq_begin,
                     int seq_end, int num_tokens, int nq, int nkv, int page_size, int num_pages, int window,
                     float scale, int* err, cudaStream_t stream) {
  const int g = nq / nkv;
  CUtensorMap mq, mk, mv;
  {
    // a box is a panel of 64 dims: x selects the panel
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)nq, (cuuint64_t)num_q_rows};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)g, (cuuint32_t)(AT_BM / g)};
    int rc = at_encode(&mq, 3, q, dims, strides, box);
    if (rc) return rc;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * nkv * page_size};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    int rc = at_encode(&mk, 2, kcache, dims, strides, box);
    if (rc) return rc;
    rc = at_encode(&mv, 2, vcache, dims, strides, box);
    if (rc) return rc;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, at_smem_bytes<D>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int bq = AT_BM / g;
  const long long tiles = (num_tokens + bq - 1) / bq + (seq_end - seq_begin);
  if (tiles * nkv > 0x7fffffffLL) return RLLM_E_UNSUPPORTED;
  dim3 grid((unsigned)(tiles * nkv));
  attention_tcgen05_kernel<D><<<grid, AT_THREADS, at_smem_bytes<D>(), stream>>>(mq, mk, mv, (bf16*)out, block_table, max_blocks,
      q_start, seq_lens, seq_begin, seq_end, nq, nkv, page_size, num_pages, window, scale * 1.4426950408889634f, err);
  RLLM_LAUNCH_CHECK();
  return 0;
}

// Sequences seq_begin .. seq_end-1 of the step; q rows q_start[s] .. q_start[s+1]-1 (num_q_rows rows of
// q exist in all); head size 64 (pages of 16, 32, 64 or 128 keys) or 128 (pages of 16, 32 or 64); nq / nkv
// up to 128 (a tile holds 128 / g tokens, rounded down).
RLLM_EXPORT int rllm_attention_prefill_tcgen05(const void* q, int q_stride, int num_q_rows, void* out,
                                               const void* kcache, const void* vcache, const int* block_table,
                                               int max_blocks, const int* q_start, const int* seq_lens,
                                               int seq_begin, int seq_end, int num_tokens, int nq, int nkv, int d,
                                               int page_size, int num_pages, int window, float scale, int* err,
                                               cudaStream_t stream) {
  if (seq_end <= seq_begin || num_tokens <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv || num_pages <= 0 || max_blocks <= 0 || window < 0 || !(scale > 0.f) || !err)
    return RLLM_E_BADARG;
  const int g = nq / nkv;
  if (!(d == 64 || d == 128) || !(page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128) ||
      page_size > 8192 / d || g > AT_BM || q_stride % 8 ||
      (((uintptr_t)q | (uintptr_t)kcache | (uintptr_t)vcache) & 15))
    return RLLM_E_UNSUPPORTED;
  if ((long long)num_pages * nkv * page_size > 0x7fffffffLL) return RLLM_E_UNSUPPORTED;   // cache rows are TMA coordinates
#define AT_LAUNCH(DD) return at_launch<DD>(q, q_stride, num_q_rows, out, kcache, vcache, block_table, max_blocks, q_start, \
      seq_lens, seq_begin, seq_end, num_tokens, nq, nkv, page_size, num_pages, window, scale, err, stream)
  if (d == 64) AT_LAUNCH(64);
  AT_LAUNCH(128);
}
