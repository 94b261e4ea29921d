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
// features and stores silu(gate) * up (crates/rllm-model/src/layers.rs:214-220),
// or residual: the float32 accumulators are added to the float32 residual
// stream h in place (a CTA owns its 16 columns).
//
// The residual epilogue also prepares the RMSNorm that reads h next
// (crates/rllm-model/src/layers.rs:133-140: y = h / sqrt(mean(h^2) + eps) * w,
// float32), so that no norm kernel stands between this product and the one
// after the norm (up to 16 rows): it stores scaled[m][n] = bfloat16(h[m][n] *
// w[n]) and, for every row, the sum of squares of the CTA's 16 new values of h.
// The product that follows takes `scaled` as its operand and, told so (RSTD),
// adds up a row's partial sums in a fixed order and multiplies row m of its
// result by 1 / sqrt(mean(h[m]^2) + eps).
#include "common.cuh"
#include <stdlib.h>

#define EPI_BF16 0
#define EPI_F32 1
#define EPI_SILU 2
#define EPI_RESID 3
#define RLLM_NO_EARLY_LAUNCH 0x7fffffff     // tail_from: no CTA calls pdl_launch; the next kernel starts when this one ends

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
// RSTD: the rows' partial sums of squares; EPI_RESID: where the partial sums and the scaled copy of h go
struct NormSide {
  const float* parts; int P; float eps; int width;      // in:  [P, M]; the row's mean is over `width` values
  float* parts_out;                                     // out: [gridDim.x, M]
  const void* w_next; int w_is_f32;                     // out: weight [N] of the norm that reads h next (or null)
  bf16* scaled; int lds;                                // out: [M, N] = bfloat16(h * w_next)
};

// The parts of row m = tid % R (R = 8 MT rows) that fall to this thread's slice tid / R, added in order; the
// loads are independent of one another.  Rows past M repeat the last row.  (The kernel ahead wrote them: the
// caller passes a pointer made behind the wait, see pdl_fresh.)
template <int R>
__device__ __forceinline__ float rows_sumsq_slice(const float* __restrict__ parts, int P, int M) {
  const int m = min((int)(threadIdx.x % R), M - 1), slice = threadIdx.x / R, nslices = blockDim.x / R;
  float v[8], acc = 0.f;
  for (int p0 = slice; p0 < P; p0 += 8 * nslices) {          // eight loads in flight: one latency for up to 8 x nslices parts
#pragma unroll
    for (int j = 0; j < 8; ++j) { const int pp = p0 + j * nslices; v[j] = pp < P ? parts[(size_t)pp * M + m] : 0.f; }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += v[j];
  }
  return acc;
}

// Element idx = tid of the CTA's [16 columns][8 MT rows] tile of h, fetched long before it is needed.
__device__ __forceinline__ float resid_old(const void* h, int ldh, int n0, int M, int N, int MT) {
  const int cols = 8 * MT, idx = threadIdx.x;
  if (idx >= 16 * cols) return 0.f;
  const int r = idx / cols, m = idx - r * cols, n = n0 + r;
  return (m < M && n < N) ? ((const float*)h)[(size_t)m * ldh + n] : 0.f;
}

// 122 to 128 registers a thread: a CTA of 512 threads has its SM's registers to itself (the kernel behind
// it comes in on the SMs that the grid leaves free and where CTAs have ended), two CTAs of 256 threads
// likewise; a single CTA of 256 threads leaves half an SM to the CTAs of its neighbours in the stream.
// UMAX = 4 (88 registers with the residual epilogue): for warps with at most four k blocks, see the launch.
// LIGHT: half as many loads in flight a thread and at most 73 registers, so that seven CTAs of four warps
// fit on an SM: for grids that then run as one wave where the ordinary form needs two, the second of them
// three quarters empty.
template <int MT, int EPI, bool RSTD, bool LIGHT = false, int UMAX = 8>
__global__ void __launch_bounds__(LIGHT ? 128 : 512, LIGHT ? 7 : 1)
gemm_small_m_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ W, int ldw,
                    void* __restrict__ out, int ldo, int M, int N, int K, int up_offset, int tail_from,
                    NormSide ns) {
  extern __shared__ float red[];                 // [warps][16][8 MT]
  __shared__ float s_rstd[8 * MT];
  __shared__ float s_part[RSTD ? 512 : 1];          // [slices][8 MT], one value a thread
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
  constexpr int U0 = LIGHT ? (MT == 1 ? 4 : 2) : (MT == 1 ? 8 : (MT == 2 ? 4 : 2));
  constexpr int U = U0 < UMAX ? U0 : UMAX;       // (UMAX: a warp has no more k blocks than that, see the launch)
  // a warp takes a contiguous range of k blocks, so that its loads walk along the rows of W
  const int per_warp = (nblocks + nwarps - 1) / nwarps;
  const int b_end = min(nblocks, (warp + 1) * per_warp);
  bool waited = false;
  // RSTD: thread (slice, m) = (tid / 8, tid % 8) adds the parts slice, slice + nslices, ... of row m
  float psum = 0.f;
  bool summed = false;
  // EPI_RESID: the old value of the element of h that this thread will update (threads 0 .. 16 * 8 MT - 1)
  float h_old = 0.f;
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
    const bool first = !waited;
    if (first) {
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
    // What else the kernel before this one wrote: behind the loads of x.  The norm's partial sums wait for the
    // warp's second round of loads where it has one: they are then fetched and added while weights are on
    // their way, and the first multiplies do not wait for them.
    if (first && EPI == EPI_RESID) h_old = resid_old(out, ldo, n0, M, N, MT);
    if (RSTD && !summed && (!first || b0 + U >= b_end)) {
      psum = rows_sumsq_slice<8 * MT>(pdl_fresh(ns.parts), ns.P, M);
      summed = true;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        mma16816(c[i], a[u].x, v[u].x, a[u].y, v[u].y, xb[u][i].x, xb[u][i].y);
        mma16816(c[i], a[u].z, v[u].z, a[u].w, v[u].w, xb[u][i].z, xb[u][i].w);
      }
  }
  if (!waited) {                 // a warp without k blocks: nothing was read, but what follows must wait too
    pdl_wait();
    if (EPI == EPI_RESID) h_old = resid_old(out, ldo, n0, M, N, MT);
  }
  if (tail_from != RLLM_NO_EARLY_LAUNCH) pdl_launch();   // the stream's next kernel may start coming in now
  // partial sums of the warps -> shared memory; c[i]: rows gq, gq + 8; batch columns i*8 + 2t, 2t + 1
  float* mine = red + (size_t)warp * 16 * 8 * MT;
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    mine[gq * 8 * MT + i * 8 + 2 * t] = c[i][0];
    mine[gq * 8 * MT + i * 8 + 2 * t + 1] = c[i][1];
    mine[(gq + 8) * 8 * MT + i * 8 + 2 * t] = c[i][2];
    mine[(gq + 8) * 8 * MT + i * 8 + 2 * t + 1] = c[i][3];
  }
  if (RSTD) {
    if (!summed) psum = rows_sumsq_slice<8 * MT>(pdl_fresh(ns.parts), ns.P, M);
    s_part[threadIdx.x] = psum;
    __syncthreads();
    if (threadIdx.x < 8 * MT) {
      float ss = 0.f;
      for (int sl = 0; sl < (int)(blockDim.x / (8 * MT)); ++sl) ss += s_part[sl * 8 * MT + threadIdx.x];
      s_rstd[threadIdx.x] = 1.0f / sqrtf(ss / (float)ns.width + ns.eps);     // eps inside the root
    }
  }
  __syncthreads();
  const int cols = 8 * MT;
  if (EPI == EPI_RESID) {
    // h[m][n] += acc for the CTA's 16 columns n; the scaled copy; then, row by row, the sum of squares
    float* tile = red + (size_t)nwarps * 16 * cols;          // [8 MT][16] new values of h (0 outside the matrix)
    for (int idx = threadIdx.x; idx < 16 * cols; idx += blockDim.x) {
      const int r = idx / cols, m = idx - r * cols;
      float acc = 0.f;
      for (int w = 0; w < nwarps; ++w) acc += red[((size_t)w * 16 + r) * cols + m];
      const int n = n0 + r;
      float hv = 0.f;
      if (m < M && n < N) {
        float* hp = (float*)out + (size_t)m * ldo + n;
        hv = (idx == (int)threadIdx.x ? h_old : *hp) + acc;      // blocks of fewer than 16 * cols threads: later elements are read here
        *hp = hv;
        if (ns.scaled) {
          const float wv = ns.w_is_f32 ? ((const float*)ns.w_next)[n] : __bfloat162float(((const bf16*)ns.w_next)[n]);
          ns.scaled[(size_t)m * ns.lds + n] = __float2bfloat16_rn(hv * wv);
        }
      }
      tile[m * 16 + r] = hv;
    }
    __syncthreads();
    if (threadIdx.x < cols && threadIdx.x < M) {
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < 16; ++r) { const float v = tile[threadIdx.x * 16 + r]; ss += v * v; }
      ns.parts_out[(size_t)blockIdx.x * M + threadIdx.x] = ss;
    }
  } else if (EPI == EPI_SILU) {
    for (int idx = threadIdx.x; idx < 8 * cols; idx += blockDim.x) {
      const int r = idx / cols, m = idx - r * cols;
      float g = 0.f, u = 0.f;
      for (int w = 0; w < nwarps; ++w) {
        g += red[((size_t)w * 16 + r) * cols + m];
        u += red[((size_t)w * 16 + r + 8) * cols + m];
      }
      const int n = n0 + r;
      if (RSTD) { g *= s_rstd[m]; u *= s_rstd[m]; }
      if (m < M && n < N) ((bf16*)out)[(size_t)m * ldo + n] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
    }
  } else {
    for (int idx = threadIdx.x; idx < 16 * cols; idx += blockDim.x) {
      const int r = idx / cols, m = idx - r * cols;
      float acc = 0.f;
      for (int w = 0; w < nwarps; ++w) acc += red[((size_t)w * 16 + r) * cols + m];
      const int n = n0 + r;
      if (RSTD) acc *= s_rstd[m];
      if (m < M && n < N) {
        if (EPI == EPI_F32) ((float*)out)[(size_t)m * ldo + n] = acc;
        else ((bf16*)out)[(size_t)m * ldo + n] = __float2bfloat16_rn(acc);
      }
    }
  }
}

template <int MT, int EPI, bool RSTD>
static int launch_small_m(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo, int M, int N, int K,
                          int up_offset, NormSide ns, cudaStream_t stream) {
  const int rows_per_cta = (EPI == EPI_SILU) ? 8 : 16;
  const int tiles = (N + rows_per_cta - 1) / rows_per_cta;
  const int nblocks = (K + 31) / 32;
  // More warps a CTA (K split further) while there are few tiles, but only as long as the whole grid stays
  // resident at once: 512 threads fit on an SM, and a second wave of a few CTAs costs as much as a full one
  // (320 tiles of 8 warps: 296 at once and then 24 alone, 12 us where 4 warps take 8).
  static int sms = 0;
  if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); if (sms <= 0) sms = 148; }
  int warps = 4;
  while (warps < 16 && (long long)tiles * warps < 1536 && tiles <= (16 / (2 * warps)) * sms) warps *= 2;
  // One or two rows, a short K (the o projection of a small model): eight warps with eight k blocks each are
  // ahead of sixteen with four (batch 1 at the Llama-3.2-1B shape: 1,630 against 1,598 tok/s; no difference
  // that the clock could see at batch 8).
  if (EPI == EPI_RESID && M <= 2 && warps == 16 && nblocks <= 64) warps = 8;
  while (warps > 1 && warps > nblocks) warps /= 2;
  while (warps > 1 && (size_t)warps * 16 * 8 * MT * sizeof(float) > 40 * 1024) warps /= 2;
  // EPI_RESID keeps the CTA's new values of h behind the warps' partial sums
  const size_t smem = ((size_t)warps * 16 * 8 * MT + (EPI == EPI_RESID ? 16 * 8 * MT : 0)) * sizeof(float);
  static int resident[17];       // by number of warps
  if (!resident[warps]) resident[warps] = rllm_resident_ctas(gemm_small_m_kernel<MT, EPI, RSTD>, 32 * warps, smem) + 1;
  int tail_from = resident[warps] > 1 ? tiles - (resident[warps] - 1) : tiles;
  // A product with a small weight (the o projection of a small model) is over in a few microseconds, all
  // of them latency.  Measured at 3 to 8 rows: when it lets the large product behind it in while it runs,
  // the step takes 13 % longer than when that product starts at its end; so it lets nothing in early.
  const size_t weight_bytes = (size_t)(EPI == EPI_SILU ? 2 : 1) * N * K * sizeof(bf16);
  if (weight_bytes < ((size_t)12 << 20) && M > 2) tail_from = RLLM_NO_EARLY_LAUNCH;
  if (MT <= 2 && warps == 4 && tiles >= resident[warps]) {
    static int light = 0;
    if (!light) {
      light = rllm_resident_ctas(gemm_small_m_kernel<MT, EPI, RSTD, true>, 128, smem) + 1;
      const char* env = getenv("RLLM_SMALL_M_LIGHT");
      if (env && env[0] == '0') light = 1;
    }
    if (tiles < light) {      // one wave: every CTA is there from the start
      if (tail_from != RLLM_NO_EARLY_LAUNCH) tail_from = 0;
      cudaError_t e = rllm_launch_pdl(gemm_small_m_kernel<MT, EPI, RSTD, true>, dim3(tiles), dim3(128), smem, stream,
                                      x, ldx, W, ldw, out, ldo, M, N, K, up_offset, tail_from, ns);
      return (int)e;
    }
  }
  // A warp with at most four k blocks (the o projection of a small model: 64 blocks over 16 warps) needs no room
  // for eight: with the registers of four, a CTA of 512 threads leaves room on its SM for a CTA of the kernel
  // ahead that is still running, and comes in beside it instead of behind it.
  // (batch 1 at the Llama-3.2-1B shape: 1,545 against 1,530 tok/s; batch 8 the same within its spread)
  if constexpr (EPI == EPI_RESID && MT == 1) if ((nblocks + warps - 1) / warps <= 4) {
    cudaError_t e4 = rllm_launch_pdl(gemm_small_m_kernel<MT, EPI, RSTD, false, 4>, dim3(tiles), dim3(32 * warps), smem, stream,
                                     x, ldx, W, ldw, out, ldo, M, N, K, up_offset, tail_from, ns);
    return (int)e4;
  }
  cudaError_t e = rllm_launch_pdl(gemm_small_m_kernel<MT, EPI, RSTD>, dim3(tiles), dim3(32 * warps), smem, stream,
                                  x, ldx, W, ldw, out, ldo, M, N, K, up_offset, tail_from, ns);
  if (e != cudaSuccess) return (int)e;
  return 0;
}

template <int EPI>
static int dispatch_mt(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo, int M, int N, int K,
                       int up_offset, cudaStream_t stream) {
  NormSide none = {};
  if (M <= 8) return launch_small_m<1, EPI, false>(x, ldx, W, ldw, out, ldo, M, N, K, up_offset, none, stream);
  if (M <= 16) return launch_small_m<2, EPI, false>(x, ldx, W, ldw, out, ldo, M, N, K, up_offset, none, stream);
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

// How many partial sums a row gets from rllm_gemm_small_m_residual with N columns.
RLLM_EXPORT int rllm_gemm_small_m_parts(int N) { return (N + 15) / 16; }

// h[M, N] (float32, in place) += x[M, K] . W[N, K]^T for M <= 16 rows.  parts_out
// [rllm_gemm_small_m_parts(N), M] receives, part by part, the sums of squares of 16 new values of each
// row; with w_next (weight [N] of the norm that reads h next, float32 or bfloat16), scaled [M, N] receives
// bfloat16(h * w_next).
RLLM_EXPORT int rllm_gemm_small_m_residual(const void* x, int ldx, const void* W, int ldw, float* h, int ldh,
                                           float* parts_out, const void* w_next, int w_is_f32, void* scaled,
                                           int lds, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || ldx < K || ldw < K || ldh < N || !parts_out || (scaled && (!w_next || lds < N))) return RLLM_E_BADARG;
  if (K % 8 || ldx % 8 || ldw % 8 || M > 16) return RLLM_E_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return RLLM_E_BADARG;
  NormSide ns = {};
  ns.parts_out = parts_out; ns.w_next = w_next; ns.w_is_f32 = w_is_f32; ns.scaled = (bf16*)scaled; ns.lds = lds;
  if (M <= 8) return launch_small_m<1, EPI_RESID, false>((const bf16*)x, ldx, (const bf16*)W, ldw, h, ldh, M, N, K, 0, ns, stream);
  return launch_small_m<2, EPI_RESID, false>((const bf16*)x, ldx, (const bf16*)W, ldw, h, ldh, M, N, K, 0, ns, stream);
}

// out = (x . W^T) with row m scaled by 1 / sqrt(sum_p parts[p][m] / K + eps), for M <= 16 rows: x is the
// `scaled` output of rllm_gemm_small_m_residual and parts [P, M] its partial sums, so that out is the
// product of the RMS-normalised h with W.  epilogue 0 (bfloat16 out) or 2 (SiLU-gate), as above.
RLLM_EXPORT int rllm_gemm_small_m_rstd(const void* x, int ldx, const float* parts, int P, float eps, const void* W,
                                       int ldw, void* out, int ldo, int M, int N, int K, int epilogue,
                                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || ldx < K || ldw < K || ldo < N || P <= 0 || !parts || !(eps > 0.f)) return RLLM_E_BADARG;
  if (K % 8 || ldx % 8 || ldw % 8 || M > 16) return RLLM_E_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return RLLM_E_BADARG;
  NormSide ns = {};
  ns.parts = parts; ns.P = P; ns.eps = eps; ns.width = K;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
  if (M <= 8) {
    if (epilogue == EPI_BF16) return launch_small_m<1, EPI_BF16, true>(xp, ldx, wp, ldw, out, ldo, M, N, K, 0, ns, stream);
    if (epilogue == EPI_SILU) return launch_small_m<1, EPI_SILU, true>(xp, ldx, wp, ldw, out, ldo, M, N, K, N, ns, stream);
  } else {
    if (epilogue == EPI_BF16) return launch_small_m<2, EPI_BF16, true>(xp, ldx, wp, ldw, out, ldo, M, N, K, 0, ns, stream);
    if (epilogue == EPI_SILU) return launch_small_m<2, EPI_SILU, true>(xp, ldx, wp, ldw, out, ldo, M, N, K, N, ns, stream);
  }
  return RLLM_E_BADARG;
}
