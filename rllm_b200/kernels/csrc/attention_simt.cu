// Paged causal attention on CUDA cores, for float32 and bfloat16 caches: the
// kernel of the true 32-bit path, and the fallback of the bfloat16 path for
// shapes its tensor-core kernels refuse.  One warp per (query token, query
// head); it serves prompt portions and single decoded tokens alike, since a
// token's keys are read from the cache through the block table either way.
//
// Contract (the reference's intended one, crates/rllm-kernels/src/cuda/
// paged_attention.cu:88-179 for the math; its prefill kernel ignores earlier
// context at :285-286, which this does not): the query at position p of
// sequence s sees keys max(0, p - window + 1) .. p of s (window 0: all keys
// 0 .. p); kv head of query head h is h / (nq / nkv) (:113); scores are
// scaled by `scale`; softmax is online in float32 (:159-169), P.V is
// accumulated in float32 and divided by the sum once (:173-178).
//
// Keys are walked in groups of 32 aligned to absolute positions, so the
// arithmetic of a row does not depend on how the sequence was cut into steps,
// on the batch around it, or on which pages hold it.
#include "common.cuh"
#include <math.h>

#define ATT_WARPS 4
#define ATT_MAX_D 256

template <typename T> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* o) {
    float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  }
};
template <> struct Vec8<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float* o) {
    uint4 a = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&a;
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
  }
};

template <typename T>
__global__ void __launch_bounds__(32 * ATT_WARPS)
attention_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                      const T* __restrict__ kcache, const T* __restrict__ vcache,
                      const int* __restrict__ block_table, int max_blocks,
                      const int* __restrict__ positions, const int* __restrict__ token_seq, int T_tokens,
                      int nq, int nkv, int d, int page_size, int num_pages, int window, float scale,
                      int* __restrict__ err) {
  extern __shared__ float qs[];  // [ATT_WARPS][d]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long gw = (long long)blockIdx.x * ATT_WARPS + warp;
  if (gw >= (long long)T_tokens * nq) return;
  const int t = (int)(gw / nq), h = (int)(gw - (long long)t * nq);
  const int kvh = h / (nq / nkv);
  const int s = token_seq[t];
  const int qpos = positions[t];
  const int kend = qpos + 1;
  const int kstart = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
  float* myq = qs + warp * d;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) myq[i] = to_f32(qrow[i]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_D / 32];
#pragma unroll
  for (int r = 0; r < ATT_MAX_D / 32; ++r) acc[r] = 0.f;
  const int* bt = block_table + (size_t)s * max_blocks;

  for (int j0 = (kstart / 32) * 32; j0 < kend; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = (j >= kstart) && (j < kend);
    float score = -INFINITY;
    int page = -1;
    if (valid) {
      page = bt[j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, 4);
        page = -1;
      } else {
        const T* kp = kcache + (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * d;
        float dot = 0.f;
        for (int i = 0; i < d; i += 8) {
          float kv[8];
          Vec8<T>::load(kp + i, kv);
#pragma unroll
          for (int u = 0; u < 8; ++u) dot = fmaf(myq[i + u], kv[u], dot);
        }
        score = dot * scale;
      }
    }
    const float cmax = warp_max(score);
    const float m_new = fmaxf(m, cmax);
    if (m_new == -INFINITY) continue;  // nothing visible in this group (warp-uniform)
    const float p = (score == -INFINITY) ? 0.f : expf(score - m_new);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int r = 0; r < ATT_MAX_D / 32; ++r) acc[r] *= corr;
    m = m_new;
    const int jn = min(32, kend - j0);
    for (int jj = max(0, kstart - j0); jj < jn; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int pg = __shfl_sync(0xffffffffu, page, jj);
      if (pg < 0) continue;
      const T* vp = vcache + (((size_t)pg * nkv + kvh) * page_size + ((j0 + jj) % page_size)) * d;
#pragma unroll
      for (int r = 0; r < ATT_MAX_D / 32; ++r) {
        const int i = lane + 32 * r;
        if (i < d) acc[r] = fmaf(pj, to_f32(vp[i]), acc[r]);
      }
    }
  }
  T* orow = out + ((size_t)t * nq + h) * d;
  const float inv = (l > 0.f) ? 1.0f / l : 0.f;
#pragma unroll
  for (int r = 0; r < ATT_MAX_D / 32; ++r) {
    const int i = lane + 32 * r;
    if (i < d) orow[i] = from_f32<T>(acc[r] * inv);
  }
}

RLLM_EXPORT int rllm_attention_simt(const void* q, int q_stride, void* out, const void* kcache,
                                    const void* vcache, int dtype, const int* block_table,
                                    int max_blocks, const int* positions, const int* token_seq, int T,
                                    int nq, int nkv, int d, int page_size, int num_pages, int window,
                                    float scale, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || d <= 0 || page_size <= 0 || num_pages <= 0 ||
      max_blocks <= 0 || window < 0)
    return RLLM_E_BADARG;
  if (d % 16 != 0 || d > ATT_MAX_D) return RLLM_E_UNSUPPORTED;  // head sizes in steps of 16, to 256
  if (q_stride % 8 != 0) return RLLM_E_BADARG;
  const long long warps = (long long)T * nq;
  const unsigned blocks = (unsigned)((warps + ATT_WARPS - 1) / ATT_WARPS);
  const size_t smem = (size_t)ATT_WARPS * d * sizeof(float);
  RLLM_DISPATCH_DTYPE(dtype, T_,
    (attention_simt_kernel<T_><<<blocks, 32 * ATT_WARPS, smem, stream>>>(
        (const T_*)q, q_stride, (T_*)out, (const T_*)kcache, (const T_*)vcache, block_table,
        max_blocks, positions, token_seq, T, nq, nkv, d, page_size, num_pages, window, scale, err)));
  RLLM_LAUNCH_CHECK();
  return 0;
}
