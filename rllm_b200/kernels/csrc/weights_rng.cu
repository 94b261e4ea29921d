// Random weights that are the same wherever they are drawn.
//
// Element i of a tensor is a function of (key, i) alone: Philox4x32-10 with the 64-bit key of the tensor
// (model seed and a hash of the tensor's name) and the counter i / 4 gives four 32-bit words; words (0, 1)
// and (2, 3) each make a pair of standard normals by the Box-Muller transform; element i takes normal
// number i % 4.  The transform is written out in IEEE double arithmetic with additions, multiplications,
// divisions and one square root only, each rounded once (no fused multiply-add, no library logarithm or
// cosine), so that the NumPy twin in rllm_b200/weights/counter_rng.py, which performs the same operations
// in the same order, produces the same bits.  The reference has only an unseeded test helper
// (crates/rllm-model/src/llama.rs:367-428).
//
//   u   = (w0 + 0.5) / 2^32 in (0, 1)        r = sqrt(-2 ln u)
//   phi = 2 pi w1 / 2^32                     z0 = r cos phi, z1 = r sin phi
//   ln u:  u = m 2^e with m in [sqrt(1/2), sqrt(2)),  s = (m - 1) / (m + 1),
//          ln m = 2 s (1 + s^2/3 + s^4/5 + ... + s^26/27)     (|s| < 0.172: the next term is below 1e-21)
//   cos, sin: the top three bits of w1 name the octant, the other 29 the angle t in [0, pi/4) inside it,
//          Taylor polynomials to t^16 and t^17 (below 3e-18), then the octant's reflection.
#include "common.cuh"

namespace {

__device__ __forceinline__ void philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0,
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

// every operation rounded once, none contracted
__device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }

__device__ double ln_exact_ops(double u) {
  int e;
  double m = frexp(u, &e);                       // u = m 2^e, m in [0.5, 1): exact
  if (m < 0.70710678118654752) { m = mul(m, 2.0); e -= 1; }
  const double s = __ddiv_rn(add(m, -1.0), add(m, 1.0));
  const double s2 = mul(s, s);
  double p = 1.0 / 27.0;
#pragma unroll
  for (int k = 25; k >= 1; k -= 2) p = add(mul(p, s2), __ddiv_rn(1.0, (double)k));
  return add(mul(mul(2.0, s), p), mul((double)e, 0.69314718055994531));
}

__device__ void cos_sin_exact_ops(unsigned w, double* c, double* s) {
  const unsigned octant = w >> 29;
  const double t = mul((double)(w & 0x1FFFFFFFu), 0.78539816339744831 / 536870912.0);    // [0, pi/4)
  const double t2 = mul(t, t);
  // cos t = 1 - t^2/2! + ... + t^16/16!;  sin t = t (1 - t^2/3! + ... + t^16/17!)
  double pc = 1.0 / 20922789888000.0, ps = 1.0 / 355687428096000.0;
  const double fc[8] = {-1.0 / 87178291200.0, 1.0 / 479001600.0, -1.0 / 3628800.0, 1.0 / 40320.0, -1.0 / 720.0,
                        1.0 / 24.0, -0.5, 1.0};
  const double fs[8] = {-1.0 / 1307674368000.0, 1.0 / 6227020800.0, -1.0 / 39916800.0, 1.0 / 362880.0,
                        -1.0 / 5040.0, 1.0 / 120.0, -1.0 / 6.0, 1.0};
#pragma unroll
  for (int k = 0; k < 8; ++k) { pc = add(mul(pc, t2), fc[k]); ps = add(mul(ps, t2), fs[k]); }
  const double ct = pc, st = mul(ps, t);
  // angle = octant * pi/4 + t
  double cc, ss;
  switch (octant) {
    case 0: cc = ct; ss = st; break;
    case 1: { const double h = 0.70710678118654752; cc = mul(h, add(ct, -st)); ss = mul(h, add(ct, st)); break; }
    case 2: cc = -st; ss = ct; break;
    case 3: { const double h = 0.70710678118654752; cc = mul(h, add(-ct, -st)); ss = mul(h, add(ct, -st)); break; }
    case 4: cc = -ct; ss = -st; break;
    case 5: { const double h = 0.70710678118654752; cc = mul(h, add(st, -ct)); ss = mul(h, add(-ct, -st)); break; }
    case 6: cc = st; ss = -ct; break;
    default: { const double h = 0.70710678118654752; cc = mul(h, add(ct, st)); ss = mul(h, add(st, -ct)); break; }
  }
  *c = cc; *s = ss;
}

__device__ void normal_pair(unsigned w0, unsigned w1, double* z0, double* z1) {
  const double u = mul(add((double)w0, 0.5), 1.0 / 4294967296.0);
  const double r = __dsqrt_rn(mul(-2.0, ln_exact_ops(u)));
  double c, s;
  cos_sin_exact_ops(w1, &c, &s);
  *z0 = mul(r, c);
  *z1 = mul(r, s);
}

// kind 0: out = float(std z); 1: out = float(1 + std z)
template <typename T>
__global__ void __launch_bounds__(256)
draw_normal_kernel(T* __restrict__ out, long long n, unsigned k0, unsigned k1, double std_, int kind) {
  const long long quad = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (quad * 4 >= n) return;
  unsigned w[4];
  philox4x32_10((unsigned)quad, (unsigned)((unsigned long long)quad >> 32), 0u, 0u, k0, k1, w);
  double z[4];
  normal_pair(w[0], w[1], &z[0], &z[1]);
  normal_pair(w[2], w[3], &z[2], &z[3]);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const long long i = quad * 4 + j;
    if (i >= n) break;
    double v = mul(std_, z[j]);
    if (kind == 1) v = add(1.0, v);
    out[i] = from_f32<T>(__double2float_rn(v));      // float32 first, then the held dtype: as a written file would
  }
}

__global__ void __launch_bounds__(256)
draw_randint_kernel(int* __restrict__ out, long long n, unsigned k0, unsigned k1, unsigned high) {
  const long long quad = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (quad * 4 >= n) return;
  unsigned w[4];
  philox4x32_10((unsigned)quad, (unsigned)((unsigned long long)quad >> 32), 0u, 0u, k0, k1, w);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const long long i = quad * 4 + j;
    if (i < n) out[i] = (int)(w[j] % high);
  }
}

}  // namespace

// out: n elements of dtype (RLLM_DT_F32 / RLLM_DT_BF16); kind 0: N(0, std), 1: 1 + N(0, std)
RLLM_EXPORT int rllm_draw_normal(void* out, int dtype, long long n, unsigned long long key, double std_, int kind,
                                 cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!out || (kind != 0 && kind != 1)) return RLLM_E_BADARG;
  const long long quads = (n + 3) / 4;
  const long long blocks = (quads + 255) / 256;
  if (blocks > 0x7fffffffLL) return RLLM_E_UNSUPPORTED;
  const unsigned k0 = (unsigned)key, k1 = (unsigned)(key >> 32);
  if (dtype == RLLM_DT_F32)
    draw_normal_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float*)out, n, k0, k1, std_, kind);
  else if (dtype == RLLM_DT_BF16)
    draw_normal_kernel<bf16><<<(unsigned)blocks, 256, 0, stream>>>((bf16*)out, n, k0, k1, std_, kind);
  else
    return RLLM_E_BADARG;
  RLLM_LAUNCH_CHECK();
  return 0;
}

// out: n int32 values, word % high
RLLM_EXPORT int rllm_draw_randint(int* out, long long n, unsigned long long key, unsigned high, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!out || high == 0) return RLLM_E_BADARG;
  const long long blocks = ((n + 3) / 4 + 255) / 256;
  if (blocks > 0x7fffffffLL) return RLLM_E_UNSUPPORTED;
  draw_randint_kernel<<<(unsigned)blocks, 256, 0, stream>>>(out, n, (unsigned)key, (unsigned)(key >> 32), high);
  RLLM_LAUNCH_CHECK();
  return 0;
}
