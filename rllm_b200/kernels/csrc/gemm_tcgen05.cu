// C[M, N] = A[M, K] . W[N, K]^T in bfloat16 on the 5th-generation tensor cores
// of sm_100a: the projections of prompt portions (M > 16 rows).
//
//   * operands come from global memory by TMA (cp.async.bulk.tensor, 128-byte
//     swizzle) into a ring of shared-memory stages, signalled by mbarriers;
//   * one elected thread issues tcgen05.mma (128 x BN x 16 per instruction,
//     operands described by shared-memory matrix descriptors), accumulating in
//     float32 in tensor memory (TMEM, BN columns of the 512);
//   * tcgen05.commit hands a stage back to the TMA producer when the MMAs that
//     read it are done, and at the end tells the epilogue warps that the
//     accumulator is complete;
//   * four epilogue warps read their 32 TMEM lanes with tcgen05.ld, round to
//     bfloat16 (or keep float32) and store; with the SiLU-gate epilogue the tile
//     holds 128 gate and 128 up features of [Wgate; Wup] side by side and
//     silu(gate) * up is applied to the accumulators
//     (crates/rllm-model/src/layers.rs:214-220), so the [T, 2I] intermediate
//     never exists.
// Warp 0: TMA producer.  Warp 1: TMEM allocation and MMA issue.  Warps 2-5:
// epilogue.  The kernel is persistent (one CTA per SM walks over output tiles) and
// keeps two accumulators in TMEM, so that the epilogue of a tile overlaps the
// MMAs of the next.  No cluster, no multicast.
//
// Every wait on an mbarrier is bounded: after the limit the thread sets bit 16
// of the error word and the CTA winds down (gives its TMEM columns back) instead
// of hanging.
//
// The reference computes these products with a library call
// (crates/rllm-model/src/layers.rs:162-175).
#include "tcgen05.cuh"

#define TG_BM 128
#define TG_BK 64
#define TG_THREADS 192
#define TG_EPI_BF16 0
#define TG_EPI_F32 1
#define TG_EPI_SILU 2
template <int BN> constexpr int tg_stages() { return BN == 256 ? 4 : (BN == 192 ? 5 : 6); }
// TMEM columns for two accumulators of BN columns: a power of two
template <int BN> constexpr int tg_tmem_cols() { return BN > 128 ? 512 : 256; }
template <int BN> constexpr int tg_stage_bytes() { return (TG_BM + BN) * TG_BK * 2; }
template <int BN> constexpr int tg_smem_bytes() { return tg_stages<BN>() * tg_stage_bytes<BN>() + 1024 + 256; }

// EPI: 0 bfloat16 out, 1 float32 out, 2 SiLU-gate (BN must be 256; W rows n and up_offset + n pair up).
// Persistent: CTA b takes the output tiles b, b + gridDim.x, ... (rows of tiles first, so that CTAs
// running side by side share a weight tile in L2).  Two accumulators in TMEM: the epilogue of a
// tile runs while the tensor cores work on the next.
template <int BN, int EPI>
__global__ void __launch_bounds__(TG_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ out, int ldo, int M, int N, int K, int up_offset, int tiles_m,
                    int num_tiles, int* __restrict__ err) {
  constexpr int STAGES = tg_stages<BN>();
  constexpr int NOUT = (EPI == TG_EPI_SILU) ? BN / 2 : BN;     // output columns of a tile
  extern __shared__ unsigned char tg_raw[];
  unsigned char* base = (unsigned char*)(((uintptr_t)tg_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* stage_mem = base;
  unsigned long long* bars = (unsigned long long*)(base + STAGES * tg_stage_bytes<BN>());
  unsigned long long* full = bars;                   // [STAGES]  TMA -> MMA
  unsigned long long* empty = bars + STAGES;         // [STAGES]  MMA -> TMA
  unsigned long long* acc_full = bars + 2 * STAGES;  // [2]       MMA -> epilogue
  unsigned long long* acc_empty = acc_full + 2;      // [2]       epilogue -> MMA
  unsigned* tmem_slot = (unsigned*)(acc_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + TG_BK - 1) / TG_BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_w) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tg_smem(tmem_slot)), "r"(tg_tmem_cols<BN>()) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * TG_BM, n0 = (tile / tiles_m) * NOUT;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const unsigned phase = (it / STAGES) & 1;
          ok = mbar_wait(&empty[s], phase ^ 1, err);       // a fresh barrier passes the wait for parity 1
          if (!ok) break;
          unsigned char* sa = stage_mem + s * tg_stage_bytes<BN>();
          unsigned char* sb = sa + TG_BM * TG_BK * 2;
          mbar_expect_tx(&full[s], (unsigned)tg_stage_bytes<BN>());
          tma_load_2d(sa, &map_a, kb * TG_BK, m0, &full[s]);
          if (EPI == TG_EPI_SILU) {
            tma_load_2d(sb, &map_w, kb * TG_BK, n0, &full[s]);
            tma_load_2d(sb + (BN / 2) * TG_BK * 2, &map_w, kb * TG_BK, up_offset + n0, &full[s]);
          } else {
            tma_load_2d(sb, &map_w, kb * TG_BK, n0, &full[s]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = BN, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(TG_BM >> 4) << 24);
      unsigned it = 0, ti = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++ti) {
        const unsigned buf = ti & 1, use = ti >> 1;
        ok = mbar_wait(&acc_empty[buf], (use & 1) ^ 1, err);   // the epilogue has drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned tmem_acc = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const unsigned phase = (it / STAGES) & 1;
          ok = mbar_wait(&full[s], phase, err);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          unsigned char* sa = stage_mem + s * tg_stage_bytes<BN>();
          unsigned char* sb = sa + TG_BM * TG_BK * 2;
          const unsigned long long da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
          for (int k = 0; k < TG_BK / 16; ++k)     // 16 bf16 = 32 bytes further along K: + 2 in the address field
            umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          umma_commit(&empty[s]);                  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);       // the accumulator is complete once all MMAs are done
      }
    }
    __syncwarp();
  } else {
    // epilogue: warp w reads TMEM lanes 32 (w % 4) .. + 31 = rows of the tile
    const int quarter = warp & 3;
    unsigned ti = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++ti) {
      const int m0 = (tile % tiles_m) * TG_BM, n0 = (tile / tiles_m) * NOUT;
      const unsigned buf = ti & 1, use = ti >> 1;
      const int m = m0 + quarter * 32 + lane;
      ok = mbar_wait(&acc_full[buf], use & 1, err);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned lane_addr = tmem_base + buf * BN + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < NOUT; c0 += 32) {
        unsigned r[32];
        tmem_ld32(lane_addr + c0, r);
        if (EPI == TG_EPI_SILU) {
          unsigned u[32];
          tmem_ld32(lane_addr + NOUT + c0, u);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = __uint_as_float(r[j]);
            r[j] = __float_as_uint(__fdividef(g, 1.0f + __expf(-g)) * __uint_as_float(u[j]));
          }
        } else {
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
        if (m < M) {
          const int n = n0 + c0;
          if (EPI == TG_EPI_F32) {
            float* o = (float*)out + (size_t)m * ldo + n;
            if (n + 32 <= N && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *(float4*)(o + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            } else {
              for (int j = 0; j < 32; ++j) if (n + j < N) o[j] = __uint_as_float(r[j]);
            }
          } else {
            bf16* o = (bf16*)out + (size_t)m * ldo + n;
            if (n + 32 <= N && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 v;
                __nv_bfloat162* p = (__nv_bfloat162*)&v;
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  p[q] = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * q]), __uint_as_float(r[j + 2 * q + 1]));
                *(uint4*)(o + j) = v;
              }
            } else {
              for (int j = 0; j < 32; ++j) if (n + j < N) o[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          }
        }
      }
      // this warp has read its lanes of the accumulator: hand it back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tg_tmem_cols<BN>()) : "memory");
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
// [rows, K] bf16 row-major with row stride ld (elements); box = 64 (K) x box_rows; out-of-range reads give 0
static int tg_make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
  tg_encode_fn enc = tg_get_encode();
  if (!enc) return RLLM_E_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {TG_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : RLLM_E_BADARG;
}

// SMs of the current device (asked once per device)
static int tg_num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!cached[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 1;
  }
  return cached[dev];
}

template <int BN, int EPI>
static int tg_launch(const void* a, int lda, const void* w, int ldw, int w_rows, void* out, int ldo, int M, int N,
                     int K, int up_offset, int* err, cudaStream_t stream) {
  constexpr int NOUT = (EPI == TG_EPI_SILU) ? BN / 2 : BN;
  CUtensorMap ma, mw;
  int rc = tg_make_map(&ma, a, M, K, lda, TG_BM);
  if (rc) return rc;
  rc = tg_make_map(&mw, w, w_rows, K, ldw, NOUT);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         tg_smem_bytes<BN>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles_m = (M + TG_BM - 1) / TG_BM;
  const long long num_tiles = (long long)tiles_m * ((N + NOUT - 1) / NOUT);
  if (num_tiles > (1ll << 30)) return RLLM_E_UNSUPPORTED;
  const int num_sms = tg_num_sms();
  const int grid = (int)(num_tiles < num_sms ? num_tiles : num_sms);
  gemm_tcgen05_kernel<BN, EPI><<<grid, TG_THREADS, tg_smem_bytes<BN>(), stream>>>(ma, mw, out, ldo, M, N, K, up_offset,
                                                                                  tiles_m, (int)num_tiles, err);
  RLLM_LAUNCH_CHECK();
  return 0;
}

// epilogue 0: out bfloat16 [M, N]; 1: out float32 [M, N]; 2: W = [gate rows (N); up rows (N)] stacked,
// out bfloat16 [M, N] = silu(A . gate^T) * (A . up^T).  err: the engine's error word (bit 16: a wait ran out).
RLLM_EXPORT int rllm_gemm_tcgen05(const void* a, int lda, const void* w, int ldw, void* out, int ldo, int M, int N,
                                  int K, int epilogue, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldw < K || ldo < N || !err) return RLLM_E_BADARG;
  // TMA: 16-byte aligned bases and row strides
  if (K % 8 || lda % 8 || ldw % 8 || (((uintptr_t)a | (uintptr_t)w) & 15)) return RLLM_E_UNSUPPORTED;
  // Tile width 256, 192 or 128: the one with the least estimated time = rounds of the persistent CTAs x
  // width x a factor for what a narrower tile costs (A is read again more often, the epilogue overlaps less).
  int bn = N > 192 ? 256 : (N > 128 ? 192 : 128);
  if (N > 128) {
    const long long tm = (M + TG_BM - 1) / TG_BM, sms = tg_num_sms();
    double best = 1e30;
    const int widths[3] = {256, 192, 128};
    const double factor[3] = {1.0, 1.05, 1.3};
    for (int i = 0; i < 3; ++i) {
      const long long tiles = tm * ((N + widths[i] - 1) / widths[i]);
      const double cost = (double)((tiles + sms - 1) / sms) * widths[i] * factor[i];
      if (cost < best * 0.999) { best = cost; bn = widths[i]; }
    }
  }
#define TG_BY_WIDTH(EPI_)                                                                                      \
  if (bn == 256) return tg_launch<256, EPI_>(a, lda, w, ldw, N, out, ldo, M, N, K, 0, err, stream);            \
  if (bn == 192) return tg_launch<192, EPI_>(a, lda, w, ldw, N, out, ldo, M, N, K, 0, err, stream);            \
  return tg_launch<128, EPI_>(a, lda, w, ldw, N, out, ldo, M, N, K, 0, err, stream)
  switch (epilogue) {
    case TG_EPI_BF16: TG_BY_WIDTH(TG_EPI_BF16);
    case TG_EPI_F32: TG_BY_WIDTH(TG_EPI_F32);
    case TG_EPI_SILU:
      return tg_launch<256, TG_EPI_SILU>(a, lda, w, ldw, 2 * N, out, ldo, M, N, K, N, err, stream);
  }
  return RLLM_E_BADARG;
}
