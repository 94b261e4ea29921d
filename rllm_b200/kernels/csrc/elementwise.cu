// Memory-bound kernels of the step: embedding gather, RMSNorm fused with the
// residual add, rotary position encoding fused with the write of keys and
// values into cache pages, SiLU-gate multiply.  One source for float32 and
// bfloat16 activations; all arithmetic is float32 (rotation angles float64).
//
// The residual stream is float32 in both modes: the embedding writes it, the
// fused norm adds a block's output to it (float32 add) and hands the normed
// row on in the activation dtype.
#include "common.cuh"

// ---------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :]   (no scaling;
// crates/rllm-model/src/llama.rs:329-337)
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int H, int V, int* __restrict__ err) {
  pdl_wait_on(ids);              // (in a decode graph the token ids come from the kernel directly ahead)
  pdl_launch();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicOr(err, 1);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

RLLM_EXPORT int rllm_embedding(const int* ids, const void* table, int table_dtype, float* out,
                               int T, int H, int V, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || V <= 0) return RLLM_E_BADARG;
  int threads = H >= 1024 ? 256 : 128;
  cudaError_t e = cudaErrorInvalidValue;
  RLLM_DISPATCH_DTYPE(table_dtype, TW,
    (e = rllm_launch_pdl(embedding_kernel<TW>, dim3(T), dim3(threads), 0, stream, ids, (const TW*)table, out, H, V, err)));
  return (int)e;
}

// ---------------------------------------------------------------------------
// RMSNorm: y = x / sqrt(mean(x^2) + eps) * w   (eps inside the root, w as it
// is; crates/rllm-model/src/layers.rs:133-140).
//   x      float32 rows (the residual stream)
//   delta  optional rows in the activation dtype, added to x first (float32);
//          with writeback the sum is stored back into x
//   rows   optional row indices: output row r reads input row rows[r]
// One block per output row.  The order of the additions of a row depends on
// H and the block size only.
// ---------------------------------------------------------------------------
// four consecutive values, as one 16-byte (float) or 8-byte (bfloat16) access
__device__ __forceinline__ void load4(const float* p, float* o) {
  const float4 v = *(const float4*)p;
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
__device__ __forceinline__ void load4(const bf16* p, float* o) {
  const uint2 v = *(const uint2*)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&v.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&v.y);
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *(float4*)p = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
  uint2 v;
  *(__nv_bfloat162*)&v.x = __floats2bfloat162_rn(a, b);
  *(__nv_bfloat162*)&v.y = __floats2bfloat162_rn(c, d);
  *(uint2*)p = v;
}

template <typename TD, typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                               const int* __restrict__ rows, const TW* __restrict__ w,
                               TO* __restrict__ out, int H, float eps, int writeback, int early_launch) {
  __shared__ float red[32];
  pdl_wait_on(x, delta, rows);
  if (early_launch) pdl_launch();      // a small grid: the next kernel's CTAs find room beside it
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * H;
  const TD* dr = delta ? delta + (size_t)src * H : nullptr;
  TO* o = out + (size_t)r * H;
  float ss = 0.f;
  const bool vec = (H & 3) == 0 && ((((uintptr_t)xr | (uintptr_t)o | (uintptr_t)w) & 15) == 0) &&
                   (!dr || (((uintptr_t)dr) & 15) == 0);
  constexpr int KEEP = 4;                           // float4 values a thread keeps in registers
  const bool resident = vec && H <= 4 * KEEP * (int)blockDim.x;
  float4 kept[KEEP];
  if (resident) {
    // the row stays in registers between the two passes; 4 values a thread and step, so the
    // sums of a row keep the same order for every batch
#pragma unroll
    for (int slot = 0; slot < KEEP; ++slot) {
      const int i = (threadIdx.x + slot * blockDim.x) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < H) {
        v = *(const float4*)(xr + i);
        if (dr) {
          float d4[4];
          load4(dr + i, d4);
          v.x += d4[0]; v.y += d4[1]; v.z += d4[2]; v.w += d4[3];
          if (writeback) *(float4*)(xr + i) = v;
        }
        ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
      }
      kept[slot] = v;
    }
  } else if (vec) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 v = *(const float4*)(xr + i);
      if (dr) {
        float d4[4];
        load4(dr + i, d4);
        v.x += d4[0]; v.y += d4[1]; v.z += d4[2]; v.w += d4[3];
        if (writeback) *(float4*)(xr + i) = v;
      }
      ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i];
      if (dr) {
        v += to_f32(dr[i]);
        if (writeback) xr[i] = v;
      }
      ss += v * v;
    }
  }
  pdl_launch();
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  if (resident) {
#pragma unroll
    for (int slot = 0; slot < KEEP; ++slot) {
      const int i = (threadIdx.x + slot * blockDim.x) * 4;
      if (i < H) {
        const float4 v = kept[slot];
        float w4[4];
        load4(w + i, w4);
        store4(o + i, v.x * inv * w4[0], v.y * inv * w4[1], v.z * inv * w4[2], v.w * inv * w4[3]);
      }
    }
  } else if (vec) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 v = *(const float4*)(xr + i);
      if (dr && !writeback) {
        float d4[4];
        load4(dr + i, d4);
        v.x += d4[0]; v.y += d4[1]; v.z += d4[2]; v.w += d4[3];
      }
      float w4[4];
      load4(w + i, w4);
      store4(o + i, v.x * inv * w4[0], v.y * inv * w4[1], v.z * inv * w4[2], v.w * inv * w4[3]);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i];
      if (dr && !writeback) v += to_f32(dr[i]);
      o[i] = from_f32<TO>(v * inv * to_f32(w[i]));
    }
  }
}

template <typename TD, typename TO>
static int rmsnorm_launch_w(float* x, const void* delta, const int* rows, const void* w, int w_dtype,
                            void* out, int R, int H, float eps, int writeback, cudaStream_t stream) {
  int threads = H >= 8192 ? 1024 : (H >= 4096 ? 512 : (H >= 1024 ? 256 : (H >= 256 ? 128 : 64)));
  const int early = R <= 4 * 148 ? 1 : 0;      // all of the grid's CTAs are resident at once
  cudaError_t e;
  if (w_dtype == RLLM_DT_F32)
    e = rllm_launch_pdl(rmsnorm_kernel<TD, float, TO>, dim3(R), dim3(threads), 0, stream, x, (const TD*)delta, rows,
                        (const float*)w, (TO*)out, H, eps, writeback, early);
  else if (w_dtype == RLLM_DT_BF16)
    e = rllm_launch_pdl(rmsnorm_kernel<TD, bf16, TO>, dim3(R), dim3(threads), 0, stream, x, (const TD*)delta, rows,
                        (const bf16*)w, (TO*)out, H, eps, writeback, early);
  else
    return RLLM_E_BADARG;
  return (int)e;
}

// act_dtype is the dtype of delta and of out.
RLLM_EXPORT int rllm_rmsnorm(float* x, const void* delta, const int* rows, const void* w, int w_dtype,
                             void* out, int act_dtype, int R, int H, float eps, int writeback,
                             cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || !(eps > 0.f)) return RLLM_E_BADARG;
  if (rows && writeback) return RLLM_E_BADARG;
  if (act_dtype == RLLM_DT_F32)
    return rmsnorm_launch_w<float, float>(x, delta, rows, w, w_dtype, out, R, H, eps, writeback, stream);
  if (act_dtype == RLLM_DT_BF16)
    return rmsnorm_launch_w<bf16, bf16>(x, delta, rows, w, w_dtype, out, R, H, eps, writeback, stream);
  return RLLM_E_BADARG;
}

// x[t, :] += delta[t, :]  (float32 add), for a block's output that no norm follows.
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += to_f32(delta[i]);
}

RLLM_EXPORT int rllm_residual_add(float* x, const void* delta, int act_dtype, long long n,
                                  cudaStream_t stream) {
  if (n <= 0) return 0;
  unsigned blocks = (unsigned)((n + 255) / 256);
  RLLM_DISPATCH_DTYPE(act_dtype, TD,
    (residual_add_kernel<TD><<<blocks, 256, 0, stream>>>(x, (const TD*)delta, (size_t)n)));
  RLLM_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Rotary position encoding + write of K and V into cache pages.
//   qkv [T, (nq + 2*nkv) * d]: q heads, then k heads, then v heads of a token.
//   q is rotated in place; k is rotated and stored into its page; v is stored.
// Rotate-half convention over the first rotary_dim dims of a head
// (crates/rllm-model/src/rope.rs:57-82): for i < rd/2
//   out[i]        = x[i] * cos(p f_i) - x[i + rd/2] * sin(p f_i)
//   out[i + rd/2] = x[i + rd/2] * cos(p f_i) + x[i] * sin(p f_i)
// float32 activations: the angle p * f_i and its cosine and sine are computed in
// float64 and then rounded to float32, like the reference's table
// (rope.rs:13-31).  bfloat16 activations: the angle is reduced mod 2 pi in
// float64 and cosine and sine are float32.  The rotation itself is float32.
// rotary_dim 0 rotates nothing.
// Cache layout per layer: K and V each [num_pages, nkv, page_size, d]; token
// at position p of sequence s lies in page block_table[s][p / page_size] at
// row p % page_size (slot rule of crates/rllm-worker/src/model_runner.rs:806-826).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_seq,
                                     const double* __restrict__ inv_freq, int rotary_dim,
                                     const int* __restrict__ block_table, int max_blocks,
                                     T* __restrict__ kcache, T* __restrict__ vcache, int nq, int nkv,
                                     int d, int page_size, int num_pages, int write_kv,
                                     int* __restrict__ err) {
  extern __shared__ float cs[];  // cos[rd/2], sin[rd/2]
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rotary_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    if (sizeof(T) == 4) {            // the true 32-bit path: float64 cosine and sine, rounded once
      double a = (double)pos * inv_freq[i];
      double s, c;
      sincos(a, &s, &c);
      cs[i] = (float)c;
      cs[half + i] = (float)s;
    } else {
      rope_cos_sin(pos, inv_freq[i], &cs[i], &cs[half + i]);
    }
  }
  __syncthreads();
  T* row = qkv + (size_t)t * (nq + 2 * nkv) * d;
  // q: rotate in place
  for (int idx = threadIdx.x; idx < nq * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    T* x = row + h * d;
    const float a = to_f32(x[i]), b = to_f32(x[i + half]);
    const float c = cs[i], s = cs[half + i];
    x[i] = from_f32<T>(a * c - b * s);
    x[i + half] = from_f32<T>(b * c + a * s);
  }
  if (!write_kv) return;
  const int seq = token_seq[t];
  const int page = block_table[(size_t)seq * max_blocks + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, 2);
    return;
  }
  const int slot = pos % page_size;
  const T* ksrc = row + nq * d;
  const T* vsrc = row + (nq + nkv) * d;
  for (int idx = threadIdx.x; idx < nkv * d; idx += blockDim.x) {
    const int h = idx / d, i = idx - h * d;
    const size_t dst = (((size_t)page * nkv + h) * page_size + slot) * d + i;
    float kv = to_f32(ksrc[idx]);
    if (i < rotary_dim) {
      if (i < half) kv = kv * cs[i] - to_f32(ksrc[idx + half]) * cs[half + i];
      else          kv = kv * cs[i - half] + to_f32(ksrc[idx - half]) * cs[i];
    }
    kcache[dst] = from_f32<T>(kv);
    vcache[dst] = vsrc[idx];
  }
}

// bfloat16 with head sizes and rotary sizes that are multiples of 16: a thread takes 8 consecutive dims of
// the first half of a head's rotated part and the 8 dims that pair with them, 16 bytes a load and a store;
// the unrotated dims of k and all of v are copied 16 bytes at a time.  Same arithmetic as above.
__global__ void rope_kv_write_bf16x8_kernel(bf16* __restrict__ qkv, const int* __restrict__ positions,
                                            const int* __restrict__ token_seq,
                                            const double* __restrict__ inv_freq, int rotary_dim,
                                            const int* __restrict__ block_table, int max_blocks,
                                            bf16* __restrict__ kcache, bf16* __restrict__ vcache, int nq, int nkv,
                                            int d, int page_size, int num_pages, int write_kv,
                                            int* __restrict__ err) {
  extern __shared__ float cs[];  // cos[rd/2], sin[rd/2]
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rotary_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) rope_cos_sin(pos, inv_freq[i], &cs[i], &cs[half + i]);
  __syncthreads();
  bf16* row = qkv + (size_t)t * (nq + 2 * nkv) * d;
  long long kdst = -1;
  if (write_kv) {
    const int seq = token_seq[t];
    const int page = block_table[(size_t)seq * max_blocks + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(err, 2);
    } else {
      kdst = ((long long)page * nkv * page_size + pos % page_size) * d;     // head 0; a head further: page_size * d
    }
  }
  const int hc = half >> 3;                    // 16-byte chunks in half a rotated part
  const int heads = nq + (write_kv ? nkv : 0);
  for (int idx = threadIdx.x; idx < heads * hc; idx += blockDim.x) {
    const int h = idx / hc, c = idx - h * hc;
    bf16* x = row + (size_t)h * d + c * 8;
    const uint4 lo = *(const uint4*)x, hi = *(const uint4*)(x + half);
    const __nv_bfloat162* lp = (const __nv_bfloat162*)&lo;
    const __nv_bfloat162* hp = (const __nv_bfloat162*)&hi;
    uint4 olo, ohi;
    __nv_bfloat162* ol = (__nv_bfloat162*)&olo;
    __nv_bfloat162* oh = (__nv_bfloat162*)&ohi;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = __bfloat1622float2(lp[k]), b = __bfloat1622float2(hp[k]);
      const float c0 = cs[c * 8 + 2 * k], c1 = cs[c * 8 + 2 * k + 1];
      const float s0 = cs[half + c * 8 + 2 * k], s1 = cs[half + c * 8 + 2 * k + 1];
      ol[k] = __floats2bfloat162_rn(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
      oh[k] = __floats2bfloat162_rn(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
    }
    if (h < nq) {
      *(uint4*)x = olo;
      *(uint4*)(x + half) = ohi;
    } else if (kdst >= 0) {
      bf16* kd = kcache + kdst + (size_t)(h - nq) * page_size * d + c * 8;
      *(uint4*)kd = olo;
      *(uint4*)(kd + half) = ohi;
    }
  }
  if (kdst < 0) return;
  // the dims of k behind the rotated part, and v
  const int dc = d >> 3, rc = rotary_dim >> 3;
  for (int idx = threadIdx.x; idx < nkv * dc; idx += blockDim.x) {
    const int h = idx / dc, c = idx - h * dc;
    const size_t dst = (size_t)kdst + (size_t)h * page_size * d + c * 8;
    *(uint4*)(vcache + dst) = *(const uint4*)(row + (size_t)(nq + nkv + h) * d + c * 8);
    if (c >= rc) *(uint4*)(kcache + dst) = *(const uint4*)(row + (size_t)(nq + h) * d + c * 8);
  }
}

RLLM_EXPORT int rllm_rope_kv_write(void* qkv, int dtype, const int* positions, const int* token_seq,
                                   const double* inv_freq, int rotary_dim, const int* block_table,
                                   int max_blocks, void* kcache, void* vcache, int T, int nq, int nkv,
                                   int d, int page_size, int num_pages, int write_kv, int* err,
                                   cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nq <= 0 || nkv < 0 || d <= 0 || rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1))
    return RLLM_E_BADARG;
  if (write_kv && (page_size <= 0 || num_pages <= 0 || max_blocks <= 0)) return RLLM_E_BADARG;
  size_t smem = (size_t)rotary_dim * sizeof(float);
  if (smem > 48 * 1024) return RLLM_E_UNSUPPORTED;
  if (dtype == RLLM_DT_BF16 && d % 16 == 0 && rotary_dim % 16 == 0 && rotary_dim > 0 &&
      (((uintptr_t)qkv | (uintptr_t)kcache | (uintptr_t)vcache) & 15) == 0) {
    rope_kv_write_bf16x8_kernel<<<T, 128, smem, stream>>>((bf16*)qkv, positions, token_seq, inv_freq, rotary_dim,
        block_table, max_blocks, (bf16*)kcache, (bf16*)vcache, nq, nkv, d, page_size, num_pages, write_kv, err);
    RLLM_LAUNCH_CHECK();
    return 0;
  }
  RLLM_DISPATCH_DTYPE(dtype, T_,
    (rope_kv_write_kernel<T_><<<T, 128, smem, stream>>>((T_*)qkv, positions, token_seq, inv_freq,
        rotary_dim, block_table, max_blocks, (T_*)kcache, (T_*)vcache, nq, nkv, d, page_size,
        num_pages, write_kv, err)));
  RLLM_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// out[t, i] = silu(gu[t, i]) * gu[t, I + i],  silu(z) = z / (1 + exp(-z))
// (crates/rllm-model/src/layers.rs:214-220), float32 arithmetic.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t n) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  const float g = to_f32(gu[t * 2 * I + i]);
  const float u = to_f32(gu[t * 2 * I + I + i]);
  out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// bfloat16 with I a multiple of 8: 16-byte loads and stores, 8 values a thread
__global__ void silu_mul_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I8, size_t n8) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n8) return;
  const size_t t = idx / I8;
  const int i = (int)(idx - t * I8);
  const uint4 g = *(const uint4*)(gu + (t * 2 * I8 + i) * 8);
  const uint4 u = *(const uint4*)(gu + (t * 2 * I8 + I8 + i) * 8);
  const __nv_bfloat162* gp = (const __nv_bfloat162*)&g;
  const __nv_bfloat162* up = (const __nv_bfloat162*)&u;
  uint4 o;
  __nv_bfloat162* op = (__nv_bfloat162*)&o;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 gf = __bfloat1622float2(gp[k]), uf = __bfloat1622float2(up[k]);
    op[k] = __floats2bfloat162_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y);
  }
  *(uint4*)(out + idx * 8) = o;
}

RLLM_EXPORT int rllm_silu_mul(const void* gu, void* out, int dtype, int T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I <= 0) return RLLM_E_BADARG;
  if (dtype == RLLM_DT_BF16 && I % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
    const size_t n8 = (size_t)T * (I / 8);
    silu_mul_bf16x8_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>((const bf16*)gu, (bf16*)out, I / 8, n8);
    RLLM_LAUNCH_CHECK();
    return 0;
  }
  size_t n = (size_t)T * I;
  unsigned blocks = (unsigned)((n + 255) / 256);
  RLLM_DISPATCH_DTYPE(dtype, T_,
    (silu_mul_kernel<T_><<<blocks, 256, 0, stream>>>((const T_*)gu, (T_*)out, I, n)));
  RLLM_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Between two decode steps that stay on the device: the sampled token becomes
// the next input, positions and lengths grow by one, and the token is appended
// to a history [max_steps, S] for the host to read later.
// ---------------------------------------------------------------------------
__global__ void decode_advance_kernel(int* __restrict__ token_ids, int* __restrict__ positions,
                                      int* __restrict__ seq_lens, const int* __restrict__ sampled,
                                      int* __restrict__ history_row, int S) {
  pdl_wait_on(sampled);
  pdl_launch();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S) return;
  const int t = sampled[i];
  token_ids[i] = t;
  positions[i] += 1;
  seq_lens[i] += 1;
  if (history_row) history_row[i] = t;
}

RLLM_EXPORT int rllm_decode_advance(int* token_ids, int* positions, int* seq_lens, const int* sampled,
                                    int* history_row, int S, cudaStream_t stream) {
  if (S <= 0) return 0;
  return (int)rllm_launch_pdl(decode_advance_kernel, dim3((S + 127) / 128), dim3(128), 0, stream, token_ids, positions,
                              seq_lens, sampled, history_row, S);
}
