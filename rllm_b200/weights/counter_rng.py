"""Random tensors that are the same wherever they are drawn: on the CPU
(NumPy, this file) and on the GPU (``kernels/csrc/weights_rng.cu``).

Element i of a tensor is a function of (key, i) alone.  Philox4x32-10 with the
tensor's 64-bit key and the counter i // 4 gives four 32-bit words; words
(0, 1) and (2, 3) each make a pair of standard normals by the Box-Muller
transform; element i takes normal number i % 4.  The transform uses IEEE
double additions, multiplications, divisions and one square root only, each
rounded once, in a fixed order (logarithm by the atanh series, cosine and sine
by octant and Taylor polynomial), so both implementations give the same bits;
``tests/test_weights.py`` and ``tests/test_kernels_gpu.py`` compare them.

The reference has only an unseeded helper for its tests
(crates/rllm-model/src/llama.rs:367-428).
"""
from __future__ import annotations

import numpy as np

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_SH = np.uint64(32)


def philox4x32_10(counter: np.ndarray, key: int) -> np.ndarray:
    """uint32 [n, 4] for the 64-bit counters ``counter`` (uint64 [n]; the upper two
    counter words are zero) under the 64-bit ``key``."""
    c0 = counter & _MASK
    c1 = counter >> _SH
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = key & 0xFFFFFFFF, (key >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        n0 = (p1 >> _SH) ^ c1 ^ np.uint64(k0)
        n2 = (p0 >> _SH) ^ c3 ^ np.uint64(k1)
        c0, c1, c2, c3 = n0, p1 & _MASK, n2, p0 & _MASK
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def _ln(u: np.ndarray) -> np.ndarray:
    m, e = np.frexp(u)
    low = m < 0.70710678118654752
    m = np.where(low, m * 2.0, m)
    e = np.where(low, e - 1, e)
    s = (m + -1.0) / (m + 1.0)
    s2 = s * s
    p = np.full_like(s, 1.0 / 27.0)
    for k in range(25, 0, -2):
        p = p * s2 + 1.0 / float(k)
    return (2.0 * s) * p + e.astype(np.float64) * 0.69314718055994531


_FC = [-1.0 / 87178291200.0, 1.0 / 479001600.0, -1.0 / 3628800.0, 1.0 / 40320.0, -1.0 / 720.0, 1.0 / 24.0, -0.5, 1.0]
_FS = [-1.0 / 1307674368000.0, 1.0 / 6227020800.0, -1.0 / 39916800.0, 1.0 / 362880.0, -1.0 / 5040.0, 1.0 / 120.0,
       -1.0 / 6.0, 1.0]


def _cos_sin(w: np.ndarray):
    octant = (w >> np.uint32(29)).astype(np.int64)
    t = (w & np.uint32(0x1FFFFFFF)).astype(np.float64) * (0.78539816339744831 / 536870912.0)
    t2 = t * t
    pc = np.full_like(t, 1.0 / 20922789888000.0)
    ps = np.full_like(t, 1.0 / 355687428096000.0)
    for fc, fs in zip(_FC, _FS):
        pc = pc * t2 + fc
        ps = ps * t2 + fs
    ct, st = pc, ps * t
    h = 0.70710678118654752
    cands_c = [ct, h * (ct + -st), -st, h * (-ct + -st), -ct, h * (st + -ct), st, h * (ct + st)]
    cands_s = [st, h * (ct + st), ct, h * (ct + -st), -st, h * (-ct + -st), -ct, h * (st + -ct)]
    return np.choose(octant, cands_c), np.choose(octant, cands_s)


def _normal_pair(w0: np.ndarray, w1: np.ndarray):
    u = (w0.astype(np.float64) + 0.5) * (1.0 / 4294967296.0)
    r = np.sqrt(-2.0 * _ln(u))
    c, s = _cos_sin(w1)
    return r * c, r * s


def standard_normal(n: int, key: int) -> np.ndarray:
    """float64 [n]: the standard normals of elements 0 .. n-1 under ``key``."""
    quads = (n + 3) // 4
    out = np.empty(quads * 4, dtype=np.float64)
    step = 1 << 20                                   # bounded temporaries for large tensors
    for a in range(0, quads, step):
        b = min(quads, a + step)
        w = philox4x32_10(np.arange(a, b, dtype=np.uint64), key)
        z0, z1 = _normal_pair(w[:, 0], w[:, 1])
        z2, z3 = _normal_pair(w[:, 2], w[:, 3])
        out[4 * a:4 * b] = np.stack([z0, z1, z2, z3], axis=1).ravel()
    return out[:n]


def normal(n: int, key: int, std: float, one_plus: bool = False) -> np.ndarray:
    """float32 [n]: std * z (or 1 + std * z), computed in double and rounded once."""
    v = float(std) * standard_normal(n, key)
    if one_plus:
        v = 1.0 + v
    return v.astype(np.float32)


def randint(n: int, key: int, high: int) -> np.ndarray:
    """int32 [n]: word i of the stream modulo ``high``."""
    quads = (n + 3) // 4
    w = philox4x32_10(np.arange(quads, dtype=np.uint64), key).ravel()[:n]
    return (w % np.uint32(high)).astype(np.int32)
