// Sampling over float32 logits [R, V], one block per row, with the reference's
// pipeline (crates/rllm-sampling/src/sampler.rs:62-169): penalties and biases
// (rllm_logit_edits), masks (rllm_logit_mask), then per row: greedy when
// temperature <= 0 or top_k == 1 (:117), else temperature, top-k, top-p, min-p
// (crates/rllm-sampling/src/logits.rs:5-93) and a draw from the softmax of
// what is left (sampler.rs:194-214).
//
// Differences from the reference, on purpose:
//  * the random number of a draw comes from Philox4x32-10 keyed by the
//    request's seed with the index of the generated token as counter, so a
//    request's samples do not depend on the batch it is in (the reference
//    shares one generator between all requests and ignores the request's
//    seed, sampler.rs:37-51, 200-203);
//  * probability mass is summed in 64-bit fixed point (exp(y - max) * 2^40),
//    which is exact and independent of the order of the additions, so neither
//    the top-p cut nor the draw depends on how threads split a row;
//  * greedy ties go to the lowest index (the reference's max_by gives the
//    last, sampler.rs:184-191); top_k keeps the k largest values and their
//    ties (the reference's threshold, logits.rs:26-31, is the (k+1)-th largest,
//    which keeps k+1); top-p keeps all ties of its last value; the draw takes
//    the first index whose running sum exceeds u, so a masked token is never
//    drawn (the reference's `>=` draws index 0 when u is 0, sampler.rs:208).
#include "common.cuh"
#include <math.h>

#define SAMPLE_THREADS 1024
#define FX_ONE 1099511627776.0f  // 2^40

__device__ __forceinline__ unsigned f2key(float f) {
  unsigned b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key2f(unsigned k) {
  unsigned b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(b);
}
__device__ __forceinline__ unsigned long long fx_mass(float y, float mx) {
  return (unsigned long long)(expf(y - mx) * FX_ONE);
}

__device__ void philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0,
                              unsigned k1, unsigned* out) {
  const unsigned M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const unsigned hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const unsigned n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += W0; k1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct ArgMax { float v; int i; };
// a row's radix descent in the several-CTAs pipeline (top-k by count, then top-p by mass)
struct SelectState {
  unsigned prefix, thr_key;
  unsigned long long cum, target, total;
  int counter, active;
};
__device__ __forceinline__ ArgMax argmax_better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ ArgMax block_argmax(ArgMax a, ArgMax* sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b; b.v = __shfl_xor_sync(0xffffffffu, a.v, o); b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = argmax_better(a, b);
  }
  __syncthreads();
  if (lane == 0) sm[warp] = a;
  __syncthreads();
  ArgMax r = sm[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = argmax_better(r, sm[w]);
  return r;
}

// Radix descent over the 32-bit order keys of a row, 8 bits a pass, from the
// largest value down.  With by_mass false it finds the key of the k-th largest
// element (target = k, every element weighs 1); with by_mass true the key at
// which the mass of the elements >= it first reaches `target`.  Only elements
// with key >= floor_key take part.
__device__ unsigned radix_select(const float* __restrict__ x, int V, float inv_t, float mx,
                                 unsigned floor_key, unsigned long long target, bool by_mass,
                                 unsigned long long* hist, unsigned* sh_prefix,
                                 unsigned long long* sh_cum) {
  unsigned prefix = 0;
  unsigned long long cum = 0;  // weight of elements above the current prefix range
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0ull;
    __syncthreads();
    // The keys of a row crowd into a few bins: the lanes of a warp that hit the same bin add their
    // weights up among themselves (two 32-bit sums of the halves of weights below 2^41), and one of
    // them adds the sum to the bin.  Integer sums: the order does not matter.
    const int lane = threadIdx.x & 31;
    const int iters = (V + (int)blockDim.x - 1) / (int)blockDim.x;
    for (int it = 0; it < iters; ++it) {
      const int i = it * (int)blockDim.x + (int)threadIdx.x;
      unsigned long long w = 0;
      unsigned key = 0;
      if (i < V) {
        const float y = x[i] * inv_t;
        key = f2key(y);
        if (!(key < floor_key || (key & himask) != prefix)) w = by_mass ? fx_mass(y, mx) : 1ull;
      }
      const unsigned bin = w ? ((key >> shift) & 0xffu) : 256u + (unsigned)lane;   // lanes without weight stay alone
      const unsigned m = __match_any_sync(0xffffffffu, bin);
      if (w) {
        const unsigned lo = __reduce_add_sync(m, (unsigned)(w & 0xfffffull));
        const unsigned hi = __reduce_add_sync(m, (unsigned)(w >> 20));
        if (lane == __ffs(m) - 1) atomicAdd(&hist[bin], ((unsigned long long)hi << 20) + lo);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long c = cum;
      int b = 255;
      for (; b > 0; --b) {
        if (c + hist[b] >= target) break;
        c += hist[b];
      }
      *sh_prefix = prefix | ((unsigned)b << shift);
      *sh_cum = c;
    }
    __syncthreads();
    prefix = *sh_prefix;
    cum = *sh_cum;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const unsigned long long* __restrict__ seeds,
              const long long* __restrict__ gen_index, int* __restrict__ out_tokens) {
  __shared__ ArgMax sm_arg[32];
  __shared__ unsigned long long hist[256];
  __shared__ unsigned long long seg_sum[SAMPLE_THREADS];
  __shared__ unsigned sh_prefix;
  __shared__ unsigned long long sh_cum;
  __shared__ int sh_pick;
  const int r = blockIdx.x;
  const float* x = logits + (size_t)r * ld;
  const float temp = temperature[r];
  const int k = top_k[r];
  const bool greedy = !(temp > 0.f) || k == 1;
  const float inv_t = greedy ? 1.0f : 1.0f / temp;

  ArgMax best; best.v = -INFINITY; best.i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    ArgMax c; c.v = x[i] * inv_t; c.i = i;
    best = argmax_better(best, c);
  }
  best = block_argmax(best, sm_arg);
  if (greedy || best.v == -INFINITY) {
    if (threadIdx.x == 0) out_tokens[r] = best.i == 0x7fffffff ? 0 : best.i;
    return;
  }
  const float mx = best.v;
  unsigned thr_key = 0u;  // keep keys >= thr_key
  if (k > 0 && k < V) {
    const unsigned kk = radix_select(x, V, inv_t, mx, 0u, (unsigned long long)k, false, hist,
                                     &sh_prefix, &sh_cum);
    thr_key = max(thr_key, kk);
  }
  const float p = top_p[r];
  if (p > 0.f && p < 1.f) {
    // mass of what top-k left
    unsigned long long z = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float y = x[i] * inv_t;
      if (f2key(y) >= thr_key) z += fx_mass(y, mx);
    }
    seg_sum[threadIdx.x] = z;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long t = 0;
      for (int i = 0; i < (int)blockDim.x; ++i) t += seg_sum[i];
      sh_cum = t;
    }
    __syncthreads();
    const unsigned long long total = sh_cum;
    __syncthreads();
    unsigned long long target = (unsigned long long)((double)total * (double)p);
    if (target < 1ull) target = 1ull;
    const unsigned pk = radix_select(x, V, inv_t, mx, thr_key, target, true, hist, &sh_prefix, &sh_cum);
    thr_key = max(thr_key, pk);
  }
  const float mp = min_p[r];
  if (mp > 0.f) {
    const unsigned mk = f2key(logf(mp) + mx);
    thr_key = max(thr_key, mk);
  }
  // the draw: contiguous segment per thread, exact integer prefix sums
  const int seg = (V + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * seg, hi = min(V, lo + seg);
  unsigned long long mine = 0;
  for (int i = lo; i < hi; ++i) {
    const float y = x[i] * inv_t;
    if (f2key(y) >= thr_key) mine += fx_mass(y, mx);
  }
  seg_sum[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long total = 0;
    for (int i = 0; i < (int)blockDim.x; ++i) total += seg_sum[i];
    unsigned w[4];
    const unsigned long long seed = seeds[r];
    const unsigned long long ctr = (unsigned long long)gen_index[r];
    philox4x32_10((unsigned)ctr, (unsigned)(ctr >> 32), 0u, 0u, (unsigned)seed, (unsigned)(seed >> 32), w);
    const unsigned long long u24 = w[0] >> 8;  // u = u24 / 2^24 in [0, 1)
    const unsigned long long thi = __umul64hi(total, u24), tlo = total * u24;
    const unsigned long long target = (thi << 40) | (tlo >> 24);  // floor(total * u)
    unsigned long long c = 0;
    int pick = blockDim.x - 1;
    for (int i = 0; i < (int)blockDim.x; ++i) {
      if (c + seg_sum[i] > target) { pick = i; break; }
      c += seg_sum[i];
    }
    sh_pick = pick;
    sh_cum = target - c;  // what is left to pass inside the picked segment
  }
  __syncthreads();
  if ((int)threadIdx.x == sh_pick) {
    const unsigned long long rest = sh_cum;
    unsigned long long c = 0;
    int tok = -1, last_kept = -1;
    for (int i = lo; i < hi; ++i) {
      const float y = x[i] * inv_t;
      if (f2key(y) < thr_key) continue;
      const unsigned long long w = fx_mass(y, mx);
      if (w) last_kept = i;
      c += w;
      if (c > rest) { tok = i; break; }
    }
    if (tok < 0) tok = last_kept >= 0 ? last_kept : best.i;
    out_tokens[r] = tok;
  }
}

RLLM_EXPORT int rllm_sample_one_cta(const float* logits, int R, int V, int ld, const float* temperature,
                                    const int* top_k, const float* top_p, const float* min_p,
                                    const unsigned long long* seeds, const long long* gen_index,
                                    int* out_tokens, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) return RLLM_E_BADARG;
  sample_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, V, ld, temperature, top_k, top_p, min_p,
                                                  seeds, gen_index, out_tokens);
  RLLM_LAUNCH_CHECK();
  return 0;
}

// Greedy only: out[r] = lowest index of the largest logit of row r.  A row is cut into `split` ranges,
// one CTA each (a vocabulary of 128k in one CTA is all latency); a range's (max, index) goes to
// `partials`, and the CTA that finds itself last for its row (a counter that the kernel leaves at zero)
// takes the best of the ranges.  Ties go to the lowest index at every level, so the cut changes nothing.
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int V, int ld, int* __restrict__ out_tokens,
              ArgMax* __restrict__ partials, int* __restrict__ counters, int split) {
  __shared__ ArgMax sm_arg[32];
  __shared__ int s_last;
  pdl_wait_on(logits);
  pdl_launch();
  const int r = blockIdx.y, part = blockIdx.x;
  const float* x = logits + (size_t)r * ld;
  const int per = (((V + split - 1) / split) + 3) & ~3;
  const int lo = part * per, hi = min(V, lo + per);
  ArgMax best; best.v = -INFINITY; best.i = 0x7fffffff;
  if ((((uintptr_t)x) & 15) == 0) {
    // lo is a multiple of 4: 16-byte loads, then the tail
    const int n4 = hi > lo ? (hi - lo) >> 2 : 0;
    const float4* x4 = (const float4*)(x + lo);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 v = x4[i];
      const int j = lo + 4 * i;
      ArgMax c;
      c.v = v.x; c.i = j; best = argmax_better(best, c);
      c.v = v.y; c.i = j + 1; best = argmax_better(best, c);
      c.v = v.z; c.i = j + 2; best = argmax_better(best, c);
      c.v = v.w; c.i = j + 3; best = argmax_better(best, c);
    }
    for (int i = lo + 4 * n4 + threadIdx.x; i < hi; i += blockDim.x) {
      ArgMax c; c.v = x[i]; c.i = i;
      best = argmax_better(best, c);
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      ArgMax c; c.v = x[i]; c.i = i;
      best = argmax_better(best, c);
    }
  }
  best = block_argmax(best, sm_arg);
  if (split == 1) {
    if (threadIdx.x == 0) out_tokens[r] = best.i == 0x7fffffff ? 0 : best.i;
    return;
  }
  if (threadIdx.x == 0) {
    partials[(size_t)r * split + part] = best;
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
    const int done = atomicAdd(&counters[r], 1);
    s_last = done == split - 1;
    if (s_last) counters[r] = 0;
  }
  __syncthreads();
  if (!s_last || threadIdx.x >= 32) return;
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
  ArgMax a; a.v = -INFINITY; a.i = 0x7fffffff;
  for (int p = threadIdx.x; p < split; p += 32) {
    ArgMax c;
    c.v = __ldcg(&partials[(size_t)r * split + p].v);
    c.i = __ldcg(&partials[(size_t)r * split + p].i);
    a = argmax_better(a, c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax c; c.v = __shfl_xor_sync(0xffffffffu, a.v, o); c.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = argmax_better(a, c);
  }
  if (threadIdx.x == 0) out_tokens[r] = a.i == 0x7fffffff ? 0 : a.i;
}

// How a row of V logits is cut for rllm_argmax, and the scratch it needs: R * split (max, index) pairs of
// 8 bytes and R counters that are zero before the call (the kernel leaves them zero).
RLLM_EXPORT int rllm_argmax_split(int V) {
  const int s = (V + 4095) / 4096;
  return s < 1 ? 1 : (s > 64 ? 64 : s);
}

RLLM_EXPORT int rllm_argmax(const float* logits, int R, int V, int ld, int* out_tokens, void* partials,
                            int* counters, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V || R > 65535) return RLLM_E_BADARG;
  const int split = rllm_argmax_split(V);
  if (split > 1 && (!partials || !counters)) return RLLM_E_BADARG;
  return (int)rllm_launch_pdl(argmax_kernel, dim3(split, R), dim3(SAMPLE_THREADS), 0, stream, logits, V, ld,
                              out_tokens, (ArgMax*)partials, counters, split);
}

// ---------------------------------------------------------------------------
// The same draw with a row cut into `split` ranges, one CTA each, for rows without top-k and top-p
// (temperature and min-p only; greedy rows too): three small kernels instead of one CTA that walks a
// 128k vocabulary three times.  The mass is the same exact 64-bit fixed point, the target the same
// floor(total * u), the token the first index whose running sum exceeds it: the result is the one of
// sample_kernel, bit for bit.
//   1. sample_split_max:  (max of x / t, its lowest index) of every range
//   2. sample_split_mass: the row's max from the ranges'; the mass of every range (a greedy row is
//      finished here)
//   3. sample_split_draw: the range the target falls into, then the token inside it
// ---------------------------------------------------------------------------
__device__ __forceinline__ ArgMax row_best(const ArgMax* __restrict__ partials, int split, ArgMax* sm) {
  ArgMax a; a.v = -INFINITY; a.i = 0x7fffffff;
  for (int p = threadIdx.x; p < split; p += blockDim.x) a = argmax_better(a, partials[p]);
  return block_argmax(a, sm);
}
__device__ __forceinline__ void split_range(int V, int split, int part, int* lo, int* hi) {
  const int per = (((V + split - 1) / split) + 3) & ~3;
  *lo = min(V, part * per);
  *hi = min(V, *lo + per);
}

__global__ void __launch_bounds__(256)
sample_split_max_kernel(const float* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
                        const int* __restrict__ top_k, ArgMax* __restrict__ partials, int split) {
  __shared__ ArgMax sm_arg[32];
  pdl_wait_on(logits);
  pdl_launch();
  const int r = blockIdx.y, part = blockIdx.x;
  const float* x = logits + (size_t)r * ld;
  const float temp = temperature[r];
  const float inv_t = (!(temp > 0.f) || top_k[r] == 1) ? 1.0f : 1.0f / temp;
  int lo, hi;
  split_range(V, split, part, &lo, &hi);
  ArgMax best; best.v = -INFINITY; best.i = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    ArgMax c; c.v = x[i] * inv_t; c.i = i;
    best = argmax_better(best, c);
  }
  best = block_argmax(best, sm_arg);
  if (threadIdx.x == 0) partials[(size_t)r * split + part] = best;
}

__global__ void __launch_bounds__(256)
sample_split_mass_kernel(const float* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
                         const int* __restrict__ top_k, const float* __restrict__ min_p,
                         const ArgMax* __restrict__ partials, unsigned long long* __restrict__ psum, int split,
                         int* __restrict__ out_tokens, const SelectState* __restrict__ states) {
  __shared__ ArgMax sm_arg[32];
  __shared__ unsigned long long sm_sum[8];
  pdl_wait_on(logits, partials, states);
  pdl_launch();
  const int r = blockIdx.y, part = blockIdx.x;
  const float* x = logits + (size_t)r * ld;
  const float temp = temperature[r];
  const bool greedy = !(temp > 0.f) || top_k[r] == 1;
  const ArgMax best = row_best(partials + (size_t)r * split, split, sm_arg);
  if (greedy || best.v == -INFINITY) {
    if (part == 0 && threadIdx.x == 0) out_tokens[r] = best.i == 0x7fffffff ? 0 : best.i;
    return;
  }
  const float inv_t = 1.0f / temp, mx = best.v, mp = min_p[r];
  unsigned thr_key = mp > 0.f ? f2key(logf(mp) + mx) : 0u;
  if (states) thr_key = max(thr_key, states[r].thr_key);
  int lo, hi;
  split_range(V, split, part, &lo, &hi);
  unsigned long long mine = 0;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float y = x[i] * inv_t;
    if (f2key(y) >= thr_key) mine += fx_mass(y, mx);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if ((threadIdx.x & 31) == 0) sm_sum[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long t = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sm_sum[w];
    psum[(size_t)r * split + part] = t;
  }
}

__global__ void __launch_bounds__(256)
sample_split_draw_kernel(const float* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
                         const int* __restrict__ top_k, const float* __restrict__ min_p,
                         const unsigned long long* __restrict__ seeds, const long long* __restrict__ gen_index,
                         const ArgMax* __restrict__ partials, const unsigned long long* __restrict__ psum,
                         int split, int* __restrict__ out_tokens, const SelectState* __restrict__ states) {
  __shared__ ArgMax sm_arg[32];
  __shared__ unsigned long long seg_sum[256];
  __shared__ int sh_pick;
  __shared__ unsigned long long sh_rest;
  pdl_wait_on(logits, partials, psum, states);
  pdl_launch();
  const int r = blockIdx.x;
  const float* x = logits + (size_t)r * ld;
  const float temp = temperature[r];
  if (!(temp > 0.f) || top_k[r] == 1) return;                 // greedy: done by the kernel before
  const ArgMax best = row_best(partials + (size_t)r * split, split, sm_arg);
  if (best.v == -INFINITY) return;
  const float inv_t = 1.0f / temp, mx = best.v, mp = min_p[r];
  unsigned thr_key = mp > 0.f ? f2key(logf(mp) + mx) : 0u;
  if (states) thr_key = max(thr_key, states[r].thr_key);
  if (threadIdx.x == 0) {
    const unsigned long long* ps = psum + (size_t)r * split;
    unsigned long long total = 0;
    for (int p = 0; p < split; ++p) total += ps[p];
    unsigned w[4];
    const unsigned long long seed = seeds[r];
    const unsigned long long ctr = (unsigned long long)gen_index[r];
    philox4x32_10((unsigned)ctr, (unsigned)(ctr >> 32), 0u, 0u, (unsigned)seed, (unsigned)(seed >> 32), w);
    const unsigned long long u24 = w[0] >> 8;  // u = u24 / 2^24 in [0, 1)
    const unsigned long long thi = __umul64hi(total, u24), tlo = total * u24;
    const unsigned long long target = (thi << 40) | (tlo >> 24);  // floor(total * u)
    unsigned long long c = 0;
    int pick = split - 1;
    for (int p = 0; p < split; ++p) {
      if (c + ps[p] > target) { pick = p; break; }
      c += ps[p];
    }
    sh_pick = pick;
    sh_rest = target - c;                // what is left to pass inside the picked range
  }
  __syncthreads();
  int rlo, rhi;
  split_range(V, split, sh_pick, &rlo, &rhi);
  // inside the range: a contiguous segment a thread, exact integer prefix sums
  const int seg = (rhi - rlo + blockDim.x - 1) / blockDim.x;
  const int lo = min(rhi, rlo + (int)threadIdx.x * seg), hi = min(rhi, lo + seg);
  unsigned long long mine = 0;
  for (int i = lo; i < hi; ++i) {
    const float y = x[i] * inv_t;
    if (f2key(y) >= thr_key) mine += fx_mass(y, mx);
  }
  seg_sum[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long c = 0;
    const unsigned long long rest = sh_rest;
    int pick = blockDim.x - 1;
    for (int i = 0; i < (int)blockDim.x; ++i) {
      if (c + seg_sum[i] > rest) { pick = i; break; }
      c += seg_sum[i];
    }
    sh_pick = pick;
    sh_rest = rest - c;
  }
  __syncthreads();
  if ((int)threadIdx.x == sh_pick) {
    const unsigned long long rest = sh_rest;
    unsigned long long c = 0;
    int tok = -1, last_kept = -1;
    for (int i = lo; i < hi; ++i) {
      const float y = x[i] * inv_t;
      if (f2key(y) < thr_key) continue;
      const unsigned long long w = fx_mass(y, mx);
      if (w) last_kept = i;
      c += w;
      if (c > rest) { tok = i; break; }
    }
    if (tok < 0) tok = last_kept >= 0 ? last_kept : best.i;
    out_tokens[r] = tok;
  }
}

// ---------------------------------------------------------------------------
// Top-k and top-p with a row cut into ranges: the radix descent of radix_select, one kernel a pass.
// Every CTA adds the histogram of its range to the row's (integer sums: any order), and the CTA that
// finds itself last for the row takes the descent's next step.  Per row a SelectState and 256 bins.
//   select_begin   state for the top-k descent (or none)
//   select_pass x4 by count
//   select_total   the mass of what top-k left; state for the top-p descent (or none)
//   select_pass x4 by mass
//   then the ranges' masses and the draw, as above, with the state's threshold
// ---------------------------------------------------------------------------
__global__ void select_begin_kernel(int V, const float* __restrict__ temperature, const int* __restrict__ top_k,
                                    SelectState* __restrict__ states, unsigned long long* __restrict__ hist) {
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[(size_t)r * 256 + b] = 0ull;
  if (threadIdx.x == 0) {
    const float temp = temperature[r];
    const int k = top_k[r];
    SelectState st;
    st.prefix = 0u; st.thr_key = 0u; st.cum = 0ull; st.total = 0ull; st.counter = 0;
    st.active = (temp > 0.f && k > 1 && k < V) ? 1 : 0;
    st.target = (unsigned long long)(k > 0 ? k : 0);
    states[r] = st;
  }
}

// pass 0..3 of a descent; by_mass: weights are masses, else every element weighs 1
__global__ void __launch_bounds__(256)
select_pass_kernel(const float* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
                   const ArgMax* __restrict__ partials, int split, SelectState* __restrict__ states,
                   unsigned long long* __restrict__ hist, int pass, int by_mass) {
  __shared__ ArgMax sm_arg[32];
  __shared__ unsigned long long sh[256];
  __shared__ int s_last;
  pdl_wait_on(logits, partials);
  pdl_launch();
  const int r = blockIdx.y, part = blockIdx.x;
  SelectState* st = states + r;
  if (!st->active) return;
  const float* x = logits + (size_t)r * ld;
  const float inv_t = 1.0f / temperature[r];
  const float mx = by_mass ? row_best(partials + (size_t)r * split, split, sm_arg).v : 0.f;
  const unsigned prefix = st->prefix, floor_key = st->thr_key;
  const int shift = 24 - 8 * pass;
  const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
  for (int b = threadIdx.x; b < 256; b += blockDim.x) sh[b] = 0ull;
  __syncthreads();
  int lo, hi;
  split_range(V, split, part, &lo, &hi);
  const int lane = threadIdx.x & 31;
  const int iters = (hi - lo + (int)blockDim.x - 1) / (int)blockDim.x;
  for (int it = 0; it < iters; ++it) {
    const int i = lo + it * (int)blockDim.x + (int)threadIdx.x;
    unsigned long long w = 0;
    unsigned key = 0;
    if (i < hi) {
      const float y = x[i] * inv_t;
      key = f2key(y);
      if (!(key < floor_key || (key & himask) != prefix)) w = by_mass ? fx_mass(y, mx) : 1ull;
    }
    const unsigned bin = w ? ((key >> shift) & 0xffu) : 256u + (unsigned)lane;
    const unsigned m = __match_any_sync(0xffffffffu, bin);
    if (w) {
      const unsigned wl = __reduce_add_sync(m, (unsigned)(w & 0xfffffull));
      const unsigned wh = __reduce_add_sync(m, (unsigned)(w >> 20));
      if (lane == __ffs(m) - 1) atomicAdd(&sh[bin], ((unsigned long long)wh << 20) + wl);
    }
  }
  __syncthreads();
  unsigned long long* rh = hist + (size_t)r * 256;
  for (int b = threadIdx.x; b < 256; b += blockDim.x)
    if (sh[b]) atomicAdd(&rh[b], sh[b]);
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
    const int done = atomicAdd(&st->counter, 1);
    s_last = done == split - 1;
  }
  __syncthreads();
  if (!s_last) return;
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
  for (int b = threadIdx.x; b < 256; b += blockDim.x) { sh[b] = __ldcg(&rh[b]); rh[b] = 0ull; }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long c = st->cum;
    const unsigned long long target = st->target;
    int b = 255;
    for (; b > 0; --b) {
      if (c + sh[b] >= target) break;
      c += sh[b];
    }
    const unsigned np = prefix | ((unsigned)b << shift);
    st->cum = c;
    st->counter = 0;
    if (pass == 3) {
      st->thr_key = max(st->thr_key, np);
      st->prefix = 0u;
      st->cum = 0ull;
      st->active = 0;
    } else {
      st->prefix = np;
    }
  }
}

// the mass of what the top-k threshold left, and the state of the top-p descent
__global__ void __launch_bounds__(256)
select_total_kernel(const float* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
                    const int* __restrict__ top_k, const float* __restrict__ top_p,
                    const ArgMax* __restrict__ partials, int split, SelectState* __restrict__ states) {
  __shared__ ArgMax sm_arg[32];
  __shared__ unsigned long long sm_sum[8];
  pdl_wait_on(logits, partials);
  pdl_launch();
  const int r = blockIdx.y, part = blockIdx.x;
  SelectState* st = states + r;
  const float temp = temperature[r], p = top_p[r];
  if (!(temp > 0.f) || top_k[r] == 1 || !(p > 0.f && p < 1.f)) return;
  const ArgMax best = row_best(partials + (size_t)r * split, split, sm_arg);
  if (best.v == -INFINITY) return;
  const float* x = logits + (size_t)r * ld;
  const float inv_t = 1.0f / temp, mx = best.v;
  const unsigned thr_key = st->thr_key;
  int lo, hi;
  split_range(V, split, part, &lo, &hi);
  unsigned long long mine = 0;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float y = x[i] * inv_t;
    if (f2key(y) >= thr_key) mine += fx_mass(y, mx);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if ((threadIdx.x & 31) == 0) sm_sum[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long t = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sm_sum[w];
    atomicAdd(&st->total, t);
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
    const int done = atomicAdd(&st->counter, 1);
    if (done == split - 1) {
      asm volatile("fence.acq_rel.gpu;" ::: "memory");
      const unsigned long long total = *(volatile unsigned long long*)&st->total;
      unsigned long long target = (unsigned long long)((double)total * (double)p);
      if (target < 1ull) target = 1ull;
      st->target = target;
      st->prefix = 0u;
      st->cum = 0ull;
      st->counter = 0;
      st->active = 1;
    }
  }
}

// Bytes of scratch that rllm_sample needs: R * split (max, index) pairs and 64-bit sums, R states, R * 256 bins.
RLLM_EXPORT long long rllm_sample_scratch_bytes(int R, int V) {
  const long long split = rllm_argmax_split(V);
  return (long long)R * (split * 16 + (long long)sizeof(SelectState) + 256 * 8) + 256;
}

// The whole pipeline for any mix of rows (greedy, temperature, top-k, top-p, min-p): the same tokens as
// rllm_sample_one_cta, with every row worked on by `split` CTAs.
RLLM_EXPORT int rllm_sample(const float* logits, int R, int V, int ld, const float* temperature,
                            const int* top_k, const float* top_p, const float* min_p,
                            const unsigned long long* seeds, const long long* gen_index, int* out_tokens,
                            void* scratch, int with_select, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V || R > 65535 || !scratch || (((uintptr_t)scratch) & 15)) return RLLM_E_BADARG;
  const int split = rllm_argmax_split(V);
  ArgMax* partials = (ArgMax*)scratch;
  unsigned long long* psum = (unsigned long long*)(partials + (size_t)R * split);
  unsigned long long* hist = psum + (size_t)R * split;
  SelectState* states = (SelectState*)(hist + (size_t)R * 256);
  const dim3 g2(split, R), b(256);
  cudaError_t e = rllm_launch_pdl(sample_split_max_kernel, g2, b, 0, stream, logits, V, ld, temperature, top_k,
                                  partials, split);
  if (e != cudaSuccess) return (int)e;
  if (with_select) {
    e = rllm_launch_pdl(select_begin_kernel, dim3(R), b, 0, stream, V, temperature, top_k, states, hist);
    if (e != cudaSuccess) return (int)e;
    for (int pass = 0; pass < 4; ++pass) {
      e = rllm_launch_pdl(select_pass_kernel, g2, b, 0, stream, logits, V, ld, temperature, (const ArgMax*)partials,
                          split, states, hist, pass, 0);
      if (e != cudaSuccess) return (int)e;
    }
    e = rllm_launch_pdl(select_total_kernel, g2, b, 0, stream, logits, V, ld, temperature, top_k, top_p,
                        (const ArgMax*)partials, split, states);
    if (e != cudaSuccess) return (int)e;
    for (int pass = 0; pass < 4; ++pass) {
      e = rllm_launch_pdl(select_pass_kernel, g2, b, 0, stream, logits, V, ld, temperature, (const ArgMax*)partials,
                          split, states, hist, pass, 1);
      if (e != cudaSuccess) return (int)e;
    }
  }
  const SelectState* sts = with_select ? states : nullptr;
  e = rllm_launch_pdl(sample_split_mass_kernel, g2, b, 0, stream, logits, V, ld, temperature, top_k, min_p,
                      (const ArgMax*)partials, psum, split, out_tokens, sts);
  if (e != cudaSuccess) return (int)e;
  e = rllm_launch_pdl(sample_split_draw_kernel, dim3(R), b, 0, stream, logits, V, ld, temperature, top_k, min_p,
                      seeds, gen_index, (const ArgMax*)partials, (const unsigned long long*)psum, split, out_tokens,
                      sts);
  return (int)e;
}

// ---------------------------------------------------------------------------
// Penalties and biases on single logits.  One entry per (row, distinct token):
// bias is added first (logits.rs:147-154); then the repetition penalty is
// applied `count` times, dividing a positive logit and multiplying any other
// (:95-110, once per occurrence in the context like the reference's loop);
// then frequency * count and, if count > 0, presence are subtracted (:113-144).
// ---------------------------------------------------------------------------
__global__ void logit_edits_kernel(float* __restrict__ logits, int V, int ld, int n,
                                   const int* __restrict__ rows, const int* __restrict__ tokens,
                                   const int* __restrict__ counts, const float* __restrict__ bias,
                                   const float* __restrict__ rep, const float* __restrict__ freq,
                                   const float* __restrict__ pres) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const int r = rows[e], t = tokens[e], c = counts[e];
  if (t < 0 || t >= V) return;
  float* p = logits + (size_t)r * ld + t;
  float v = *p + bias[e];
  const float rp = rep[r];
  if (rp != 1.0f)
    for (int i = 0; i < c; ++i) v = v > 0.f ? v / rp : v * rp;
  if (c > 0) {
    if (freq[r] != 0.f) v -= freq[r] * (float)c;
    if (pres[r] != 0.f) v -= pres[r];
  }
  *p = v;
}

RLLM_EXPORT int rllm_logit_edits(float* logits, int V, int ld, int n, const int* rows,
                                 const int* tokens, const int* counts, const float* bias,
                                 const float* rep, const float* freq, const float* pres,
                                 cudaStream_t stream) {
  if (n <= 0) return 0;
  logit_edits_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, V, ld, n, rows, tokens, counts, bias,
                                                          rep, freq, pres);
  RLLM_LAUNCH_CHECK();
  return 0;
}

// Masks.  Row r keeps only the tokens of its sorted list allowed[allowed_start[r]
// .. allowed_start[r+1]) if that list is not empty (logits.rs:157-166); then the
// n_suppress pairs (row, token) are set to -inf (:169-181, :184-191).
__global__ void allowed_mask_kernel(float* __restrict__ logits, int V, int ld,
                                    const int* __restrict__ allowed_start,
                                    const int* __restrict__ allowed) {
  const int r = blockIdx.y;
  const int b = allowed_start[r], e = allowed_start[r + 1];
  if (e <= b) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= V) return;
  int lo = b, hi = e;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (allowed[mid] < i) lo = mid + 1; else hi = mid;
  }
  if (!(lo < e && allowed[lo] == i)) logits[(size_t)r * ld + i] = -INFINITY;
}
__global__ void suppress_kernel(float* __restrict__ logits, int V, int ld, int n,
                                const int* __restrict__ rows, const int* __restrict__ tokens) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const int t = tokens[e];
  if (t >= 0 && t < V) logits[(size_t)rows[e] * ld + t] = -INFINITY;
}

RLLM_EXPORT int rllm_logit_mask(float* logits, int R, int V, int ld, const int* allowed_start,
                                const int* allowed, int n_suppress, const int* sup_rows,
                                const int* sup_tokens, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (allowed_start) {
    dim3 grid((V + 255) / 256, R);
    allowed_mask_kernel<<<grid, 256, 0, stream>>>(logits, V, ld, allowed_start, allowed);
    RLLM_LAUNCH_CHECK();
  }
  if (n_suppress > 0) {
    suppress_kernel<<<(n_suppress + 255) / 256, 256, 0, stream>>>(logits, V, ld, n_suppress, sup_rows,
                                                                  sup_tokens);
    RLLM_LAUNCH_CHECK();
  }
  return 0;
}

// ---------------------------------------------------------------------------
// Log-probabilities (natural log) from a row of raw logits, as the reference's sampler reports them
// (crates/rllm-sampling/src/logprobs.rs:5-28: logit - (max + ln sum exp(logit - max)); :34-70: the N
// largest, in descending order).  One CTA a row; the sum is taken in a fixed order (a thread's strided
// elements in index order, then the threads in order), so a row's values do not depend on the batch.
// Ties in the top N: the lower index first (the reference's order among equals is not defined).
// A place for which nothing is left (N beyond the vocabulary, or -inf logits only) gets id -1.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS)
logprobs_kernel(const float* __restrict__ logits, int V, int ld, const int* __restrict__ tokens, int N,
                float* __restrict__ lp, int* __restrict__ top_ids, float* __restrict__ top_lp) {
  __shared__ ArgMax sm_arg[32];
  __shared__ float sm_f[32];
  pdl_wait_on(logits, tokens);
  pdl_launch();
  const int r = blockIdx.x;
  const float* x = logits + (size_t)r * ld;
  ArgMax best; best.v = -INFINITY; best.i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) { ArgMax c; c.v = x[i]; c.i = i; best = argmax_better(best, c); }
  best = block_argmax(best, sm_arg);
  const float mx = best.v;
  float s = 0.f;
  if (mx != -INFINITY)
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(x[i] - mx);
  s = block_sum(s, sm_f);
  const float log_z = mx + logf(s);
  if (threadIdx.x == 0) {
    const int t = tokens[r];
    lp[r] = (mx == -INFINITY || t < 0 || t >= V) ? -INFINITY : x[t] - log_z;
  }
  // the N largest, one pass each: the best element that comes after the last one found
  ArgMax prev; prev.v = INFINITY; prev.i = -1;
  for (int n = 0; n < N; ++n) {
    ArgMax b; b.v = -INFINITY; b.i = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = x[i];
      if (v == -INFINITY) continue;
      if (v < prev.v || (v == prev.v && i > prev.i)) { ArgMax c; c.v = v; c.i = i; b = argmax_better(b, c); }
    }
    b = block_argmax(b, sm_arg);
    const bool none = b.i == 0x7fffffff;
    if (threadIdx.x == 0) {
      top_ids[(size_t)r * N + n] = none ? -1 : b.i;
      top_lp[(size_t)r * N + n] = none ? -INFINITY : b.v - log_z;
    }
    if (none) { prev.v = -INFINITY; prev.i = 0x7fffffff; } else prev = b;
    __syncthreads();
  }
}

// lp [R]: log-probability of tokens[r] in row r; top_ids, top_lp [R, N]: the N likeliest tokens of every row
// and their log-probabilities (N may be 0).
RLLM_EXPORT int rllm_logprobs(const float* logits, int R, int V, int ld, const int* tokens, int N, float* lp,
                              int* top_ids, float* top_lp, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V || N < 0 || !tokens || !lp || (N > 0 && (!top_ids || !top_lp))) return RLLM_E_BADARG;
  return (int)rllm_launch_pdl(logprobs_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, logits, V, ld, tokens, N, lp,
                              top_ids, top_lp);
}
