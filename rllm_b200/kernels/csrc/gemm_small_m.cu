// y[M, N] = x[M, K] . W[N, K]^T for a few rows (M <= 16) in bfloat16: the
// projections of a decode step, which are bound by reading W once from HBM.
//
// The weight is the 16-row operand of mma.sync m16n8k16 (the batch is the
// 8-column operand), and both operands go from global memory straight into
// registers with 16-byte loads: a thread's 8 consecutive k of a W row serve as
// the A fragments of two k-steps, and the same 8 consecutive k of its x row as
// the two B fragments, so the k order inside a 32-wide block is permuted the
// same way on both sides and the sum is unchanged.  W is streamed with
// evict-first loads; x (a few KB) stays in L1/L2.  The warps of a CTA split K
// into contiguous ranges; their partial sums are added in warp order, so a
// row's result does not depend on M or on the rows around it.
//
// Epilogues: plain store (bfloat16 or float32), or SiLU-gate: with W = [gate
// rows; up rows], a CTA takes 8 gate rows and the 8 up rows of the same
// features and stores silu(gate) * up (crates/rllm-model/src/layers.rs:214-220).
#include "common.cuh"
#include <stdlib.h>

#define EPI_BF16 0
#define EPI_F32 1
#define EPI_SILU 2

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: batch tiles of 8 rows.  blockDim.x = 32 * warps; warp w takes a contiguous
// range of 32-wide k blocks.  K is a multiple of 8; the last block may be partial.
template <int MT, int EPI>
__global__ void __launch_bounds__(512)
gemm_small_m_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ W, int ldw,
                    void* __restrict__ out, int ldo, int M, int N, int K, int up_offset, int tail_from) {
  extern __shared__ float red[];                 // [warps][16][8 MT]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gq = lane >> 2, t = lane & 3;
  const int rows_per_cta = (EPI == EPI_SILU) ? 8 : 16;
  const int n0 = blockIdx.x * rows_per_cta;
  // the two W rows of this thread (clamped to the matrix; rows past the end are not stored)
  int r_lo, r_hi;
  if (EPI == EPI_SILU) { r_lo = min(n0 + gq, N - 1); r_hi = up_offset + r_lo; }
  else { r_lo = min(n0 + gq, N - 1); r_hi = min(n0 + gq + 8, N - 1); }
  const bf16* w_lo = W + (size_t)r_lo * ldw + t * 8;
  const bf16* w_hi = W + (size_t)r_hi * ldw + t * 8;
  const bf16* xr[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) xr[i] = x + (size_t)min(i * 8 + gq, M - 1) * ldx + t * 8;
  float c[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;

  const int nblocks = (K + 31) / 32;
  // U blocks at a time: all their loads are issued before the first multiply, so that a
  // warp has U * (2 + MT) 16-byte loads in flight
  constexpr int U = MT == 1 ? 8 : (MT == 2 ? 4 : 2);
  // a warp takes a contiguous range of k blocks, so that its loads walk along the rows of W
  const int per_warp = (nblocks + nwarps - 1) / nwarps;
  const int b_end = min(nblocks, (warp + 1) * per_warp);
  bool waited = false;
  for (int b0 = warp * per_warp; b0 < b_end; b0 += U) {
    uint4 a[U], v[U], xb[U][MT];
    // the weight first (no kernel writes it: these loads may run ahead of the kernel before this one) ...
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (b0 + u) * 32;
      const bool in = b0 + u < b_end && k + t * 8 < K;   // K is a multiple of 8: 8 values are all in or all out
      a[u] = make_uint4(0u, 0u, 0u, 0u);
      v[u] = a[u];
      if (in) { a[u] = ld_stream16(w_lo + k); v[u] = ld_stream16(w_hi + k); }
    }
    // ... then x, which the kernel before this one wrote
    if (!waited) {
      pdl_wait();
      waited = true;
      // no CTA of this grid is still to come once its last wave runs: the stream's next kernel may
      // come in and fetch its own weights while this one works
      if ((int)blockIdx.x >= tail_from) pdl_launch();
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (b0 + u) * 32;
      const bool in = b0 + u < b_end && k + t * 8 < K;
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        xb[u][i] = make_uint4(0u, 0u, 0u, 0u);
        if (in) xb[u][i] = ld_cached16(xr[i] + k);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        mma16816(c[i], a[u].x, v[u].x, a[u].y, v[u].y, xb[u][i].x, xb[u][i].y);
        mma16816(c[i], a[u].z, v[u].z, a[u].w, v[u].w, xb[u][i].z, xb[u][i].w);
      }
  }
  if (!waited) pdl_wait();       // a warp without k blocks: nothing was read, but the stores below must wait too
  pdl_launch();                  // the stream's next kernel may start coming in now
  // partial sums of the warps -> shared memory; c[i]: rows gq, gq + 8; batch columns i*8 + 2t, 2t + 1
  float* mine = red + (size_t)warp * 16 * 8 * MT;
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    mine[gq * 8 * MT + i * 8 + 2 * t] = c[i][0];
    mine[gq * 8 * MT + i * 8 + 2 * t + 1] = c[i][1];
    mine[(gq + 8) * 8 * MT + i * 8 + 2 * t] = c[i][2];
    mine[(gq + 8) * 8 * MT + i * 8 + 2 * t + 1] = c[i][3];
  }
  __syncthreads();
  const int cols = 8 * MT;
  if (EPI == EPI_SILU) {
    for (int idx = threadIdx.x; idx < 8 * cols; idx += blockDim.x) {
      const int r = idx / cols, m = idx - r * cols;
      float g = 0.f, u = 0.f;
      for (int w = 0; w < nwarps; ++w) {
        g += red[((size_t)w * 16 + r) * cols + m];
        u += red[((size_t)w * 16 + r + 8) * cols + m];
      }
      const int n = n0 + r;
      if (m < M && n < N) ((bf16*)out)[(size_t)m * ldo + n] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
    }
  } else {
    for (int idx = threadIdx.x; idx < 16 * cols; idx += blockDim.x) {
      const int r = idx / cols, m = idx - r * cols;
      float acc = 0.f;
      for (int w = 0; w < nwarps; ++w) acc += red[((size_t)w * 16 + r) * cols + m];
      const int n = n0 + r;
      if (m < M && n < N) {
        if (EPI == EPI_F32) ((float*)out)[(size_t)m * ldo + n] = acc;
        else ((bf16*)out)[(size_t)m * ldo + n] = __float2bfloat16_rn(acc);
      }
    }
  }
}

template <int MT, int EPI>
static int launch_small_m(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo, int M, int N, int K,
                          int up_offset, cudaStream_t stream) {
  const int rows_per_cta = (EPI == EPI_SILU) ? 8 : 16;
  const int tiles = (N + rows_per_cta - 1) / rows_per_cta;
  const int nblocks = (K + 31) / 32;
  int warps = 4;
  while (warps < 16 && (long long)tiles * warps < 1536) warps *= 2;
  if (const char* e = getenv("RLLM_SMALLM_WARPS")) warps = atoi(e);
  while (warps > 1 && warps > nblocks) warps /= 2;
  while (warps > 1 && (size_t)warps * 16 * 8 * MT * sizeof(float) > 48 * 1024) warps /= 2;
  const size_t smem = (size_t)warps * 16 * 8 * MT * sizeof(float);
  static int resident[17];       // by number of warps
  if (!resident[warps]) resident[warps] = rllm_resident_ctas(gemm_small_m_kernel<MT, EPI>, 32 * warps, smem) + 1;
  const int tail_from = resident[warps] > 1 ? tiles - (resident[warps] - 1) : tiles;
  cudaError_t e = rllm_launch_pdl(gemm_small_m_kernel<MT, EPI>, dim3(tiles), dim3(32 * warps), smem, stream,
                                  x, ldx, W, ldw, out, ldo, M, N, K, up_offset, tail_from);
  if (e != cudaSuccess) return (int)e;
  return 0;
}

template <int EPI>
static int dispatch_mt(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo, int M, int N, int K,
                       int up_offset, cudaStream_t stream) {
  if (M <= 8) return launch_small_m<1, EPI>(x, ldx, W, ldw, out, ldo, M, N, K, up_offset, stream);
  if (M <= 16) return launch_small_m<2, EPI>(x, ldx, W, ldw, out, ldo, M, N, K, up_offset, stream);
  return RLLM_E_UNSUPPORTED;
}

// epilogue 0: out bfloat16 [M, N]; 1: out float32 [M, N]; 2: W = [gate rows (N); up rows (N)] stacked
// (2 N rows in all), out bfloat16 [M, N] = silu(x . gate^T) * (x . up^T).
RLLM_EXPORT int rllm_gemm_small_m(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M,
                                  int N, int K, int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || ldx < K || ldw < K || ldo < N) return RLLM_E_BADARG;
  if (K % 8 || ldx % 8 || ldw % 8 || M > 16) return RLLM_E_UNSUPPORTED;   // 16-byte loads of rows
  if (((uintptr_t)x | (uintptr_t)W) & 15) return RLLM_E_BADARG;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
  switch (epilogue) {
    case EPI_BF16: return dispatch_mt<EPI_BF16>(xp, ldx, wp, ldw, out, ldo, M, N, K, 0, stream);
    case EPI_F32: return dispatch_mt<EPI_F32>(xp, ldx, wp, ldw, out, ldo, M, N, K, 0, stream);
    case EPI_SILU: return dispatch_mt<EPI_SILU>(xp, ldx, wp, ldw, out, ldo, M, N, K, N, stream);
  }
  return RLLM_E_BADARG;
}
