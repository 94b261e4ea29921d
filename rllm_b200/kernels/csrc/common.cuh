// Shared helpers of the sm_100a kernels: element types, conversions, warp and
// block reductions, and the argument checks that every entry point runs before
// it launches.  All entry points are extern "C", take raw device pointers and
// a stream, allocate nothing and return 0, a CUDA error code (> 0), or a
// negative RLLM_E* code when they refuse the sizes they were given.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define RLLM_DT_F32 0
#define RLLM_DT_BF16 1

#define RLLM_E_BADARG (-1)     // a size or pointer the kernel cannot take
#define RLLM_E_UNSUPPORTED (-2) // a legal size this build has no kernel for

#define RLLM_EXPORT extern "C" __attribute__((visibility("default")))

#define RLLM_LAUNCH_CHECK()                          \
  do {                                               \
    cudaError_t e__ = cudaGetLastError();            \
    if (e__ != cudaSuccess) return (int)e__;         \
  } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions depends only on blockDim, never on the data.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? smem32[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// cos and sin of position * inv_freq for the bfloat16 path: the angle is reduced
// mod 2 pi in float64 (exact to ~1e-11 for positions up to 2^20), then cosine
// and sine are taken in float32 (absolute error ~2e-7).  The float32 path of the
// model uses float64 sincos instead.
__device__ __forceinline__ void rope_cos_sin(int pos, double inv_freq, float* c, float* s) {
  const double a = (double)pos * inv_freq;
  const double n = rint(a * 0.15915494309189535);
  const double r = fma(-n, 6.283185307179586, a) - n * 2.4492935982947064e-16;
  sincosf((float)r, s, c);
}

// Programmatic dependent launch: a kernel lets the next kernel of the stream start
// (pdl_launch) while it is still running, and itself waits for the kernel before it
// (pdl_wait) only when it first touches memory that kernel may have written.  What a
// kernel does before pdl_wait (index arithmetic, loads of weights that no kernel
// writes) overlaps the tail of its predecessor.  pdl_wait returns when the
// predecessor has completed and its writes are visible; without a predecessor that
// was launched this way both are no-ops.
// Rule of this code base: a kernel calls pdl_launch only after its own pdl_wait.  Then,
// when a kernel starts, every kernel but the one directly ahead of it has completed, and
// what it reads before its own pdl_wait may include what those earlier kernels wrote.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// A pointer to what the kernel ahead wrote must be taken through pdl_fresh (or pdl_wait_on) after the wait.
// The "memory" clobber of the wait does not hold back loads that the compiler has proved to read memory no
// one writes during the kernel (const __restrict__ parameters: ld.global.nc, free to move): merged or
// hoisted above the wait they return what was there before the kernel ahead wrote.  (Seen once: the Q tile
// of decode attention, loaded in two branches of which one lay before the wait, came out of a graph replay
// as the step before's.)  A pointer that comes out of an asm statement behind the wait carries no such
// proof, and its loads stay behind it.
template <typename T>
__device__ __forceinline__ T* pdl_fresh(T* p) {
  asm volatile("" : "+l"(p) : : "memory");
  return p;
}
template <typename P>
__device__ __forceinline__ void pdl_fresh_in_place(P& p) {      // P: any pointer type, qualifiers and all
  asm volatile("" : "+l"(p) : : "memory");
}
template <typename... P>
__device__ __forceinline__ void pdl_wait_on(P&... ptrs) {
  pdl_wait();
  (pdl_fresh_in_place(ptrs), ...);
}

// Launch `kernel` so that it may start before the kernel ahead of it in the stream has
// finished (the kernel must call pdl_wait before it reads that kernel's output).
// RLLM_PDL=0 in the environment turns this into an ordinary launch.
#include <stdlib.h>
static inline bool rllm_pdl_enabled() {
  static int on = -1;
  if (on < 0) { const char* e = getenv("RLLM_PDL"); on = (e && e[0] == '0') ? 0 : 1; }
  return on == 1;
}
template <typename... KArgs, typename... Args>
static inline cudaError_t rllm_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = rllm_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// How many CTAs of `kernel` the GPU holds at once.  CTAs are handed out in order of block
// index, so once the last that-many CTAs of a grid have started, no CTA of it is still to
// come: such a CTA may let the next kernel in (pdl_launch) early, since that kernel's CTAs
// can only take room that this grid no longer needs.
template <typename K>
static inline int rllm_resident_ctas(K kernel, int threads, size_t smem) {
  int per_sm = 0, dev = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) return 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return per_sm * sms;
}

// Dispatch helpers ---------------------------------------------------------
#define RLLM_DISPATCH_DTYPE(code, T, ...)                    \
  do {                                                       \
    if ((code) == RLLM_DT_F32) { typedef float T; __VA_ARGS__; } \
    else if ((code) == RLLM_DT_BF16) { typedef bf16 T; __VA_ARGS__; } \
    else return RLLM_E_BADARG;                               \
  } while (0)
