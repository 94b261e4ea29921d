"""Python faces of the CUDA kernels: torch tensors in, kernel launched on the
current stream.  There is no fallback: a tensor that is not on a CUDA device,
a missing compiler or a size that a kernel refuses raises an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build

DT_F32, DT_BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt is torch.float32:
        return DT_F32
    if dt is torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("the engine's kernels run on CUDA tensors only; there is no CPU path")
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = [0]      # entry-point calls so far (each launches at least one kernel)


def _check(code: int, what: str) -> None:
    LAUNCHES[0] += 1
    if code == 0:
        return
    if code == -1:
        raise KernelError(f"{what}: refused its arguments (bad size or pointer)")
    if code == -2:
        raise KernelError(f"{what}: this size is legal but no kernel of this build takes it")
    raise KernelError(f"{what}: CUDA error {code}")


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


# ---------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor) -> None:
    """out[t] = table[ids[t]] as float32; ids int32 [T], out float32 [T, H]."""
    lib = build.load_library("elementwise")
    T, (V, H) = ids.numel(), table.shape
    assert ids.dtype is torch.int32 and out.dtype is torch.float32 and out.shape == (T, H)
    _contig(table, "table"); _contig(out, "out")
    _check(lib.rllm_embedding(_ptr(ids), _ptr(table), c_int(dtype_code(table.dtype)), _ptr(out),
                              c_int(T), c_int(H), c_int(V), _ptr(err), _stream()), "embedding")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            writeback: bool = False) -> None:
    """out = rmsnorm(x [+ delta]) * weight; x float32 [., H]; out [R, H] in the
    activation dtype.  ``writeback`` stores x + delta into x.  ``rows`` (int32
    [R]) picks the input row of each output row."""
    lib = build.load_library("elementwise")
    H = x.shape[-1]
    R = out.shape[0]
    assert x.dtype is torch.float32 and out.shape[-1] == H and weight.numel() == H
    _contig(x, "x"); _contig(out, "out"); _contig(weight, "weight")
    if delta is not None:
        assert delta.dtype is out.dtype and delta.shape == x.shape
        _contig(delta, "delta")
    if rows is not None:
        assert rows.dtype is torch.int32 and rows.numel() == R
    else:
        assert x.shape[0] == R
    _check(lib.rllm_rmsnorm(_ptr(x), _ptr(delta), _ptr(rows), _ptr(weight),
                            c_int(dtype_code(weight.dtype)), _ptr(out), c_int(dtype_code(out.dtype)),
                            c_int(R), c_int(H), c_float(eps), c_int(1 if writeback else 0), _stream()),
           "rmsnorm")


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    lib = build.load_library("elementwise")
    assert x.dtype is torch.float32 and x.shape == delta.shape
    _contig(x, "x"); _contig(delta, "delta")
    _check(lib.rllm_residual_add(_ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype)),
                                 c_longlong(x.numel()), _stream()), "residual_add")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], rotary_dim: int, block_table: Optional[torch.Tensor],
                  kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor], nq: int, nkv: int,
                  d: int, err: torch.Tensor, write_kv: bool = True) -> None:
    """Rotates q (in place) and k, stores k and v of every token into its page.

    qkv [T, (nq + 2 nkv) d]; caches [pages, nkv, page_size, d]; inv_freq float64
    [rotary_dim / 2]; block_table int32 [S, max_blocks]."""
    lib = build.load_library("elementwise")
    T = qkv.shape[0]
    assert qkv.shape[1] == (nq + 2 * nkv) * d
    _contig(qkv, "qkv")
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype is torch.float64 and inv_freq.numel() == rotary_dim // 2
    if write_kv:
        assert kcache.dtype is qkv.dtype and vcache.dtype is qkv.dtype
        assert kcache.shape == vcache.shape and kcache.shape[1] == nkv and kcache.shape[3] == d
        _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
        pages, page_size, max_blocks = kcache.shape[0], kcache.shape[2], block_table.shape[1]
    else:
        pages = page_size = max_blocks = 0
    _check(lib.rllm_rope_kv_write(_ptr(qkv), c_int(dtype_code(qkv.dtype)), _ptr(positions),
                                  _ptr(token_seq), _ptr(inv_freq), c_int(rotary_dim),
                                  _ptr(block_table), c_int(max_blocks), _ptr(kcache), _ptr(vcache),
                                  c_int(T), c_int(nq), c_int(nkv), c_int(d), c_int(page_size),
                                  c_int(pages), c_int(1 if write_kv else 0), _ptr(err), _stream()),
           "rope_kv_write")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    lib = build.load_library("elementwise")
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype is out.dtype
    _contig(gate_up, "gate_up"); _contig(out, "out")
    _check(lib.rllm_silu_mul(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(I),
                             _stream()), "silu_mul")


def attention_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor,
                   vcache: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor,
                   token_seq: torch.Tensor, nq: int, nkv: int, d: int, window: int, scale: float,
                   err: torch.Tensor) -> None:
    """Paged causal attention of T query tokens, one warp per (token, head).

    q: T rows of nq*d values with row stride q_stride (elements); out [T, nq*d]."""
    lib = build.load_library("attention_simt")
    T = out.shape[0]
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert kcache.dtype is q.dtype and out.dtype is q.dtype
    _check(lib.rllm_attention_simt(_ptr(q), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache),
                                   c_int(dtype_code(q.dtype)), _ptr(block_table),
                                   c_int(block_table.shape[1]), _ptr(positions), _ptr(token_seq),
                                   c_int(T), c_int(nq), c_int(nkv), c_int(d), c_int(kcache.shape[2]),
                                   c_int(kcache.shape[0]), c_int(window), c_float(scale), _ptr(err),
                                   _stream()), "attention_simt")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] . w[N, K]^T, float32 FFMA."""
    lib = build.load_library("gemm_f32")
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype is torch.float32 and w.dtype is torch.float32 and out.dtype is torch.float32
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib.rllm_gemm_f32(_ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out),
                             c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), _stream()), "gemm_f32")


SMALL_M_MAX = 8       # up to here the weight-streaming GEMM beats the library's on a B200 (it takes 16)
FUSED_M_MAX = 16      # up to here a step goes through the forms of it that carry the residual add and the norm
                      # (RLLM_FUSED_M_MAX in the environment overrides it, for measurements).  Measured at
                      # context 4096: batch 12 1.32 -> 1.06 ms a step, batch 16 1.39 -> 1.16 ms, against the
                      # library's products with norm and SiLU kernels between them


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: str = "store") -> None:
    """out = x . w^T for M <= 16 rows of bfloat16, bound by one read of w.
    epilogue "store": out [M, N] bfloat16 or float32.  "silu_mul": w = [gate rows;
    up rows] stacked (2 N rows), out [M, N] bfloat16 = silu(x gate^T) * (x up^T)."""
    lib = build.load_library("gemm_small_m")
    M, K = x.shape
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if epilogue == "silu_mul":
        N = w.shape[0] // 2
        assert out.dtype is torch.bfloat16 and out.shape == (M, N) and w.shape[0] == 2 * N
        code = 2
    else:
        N = w.shape[0]
        assert out.shape == (M, N)
        code = 1 if out.dtype is torch.float32 else 0
        assert out.dtype in (torch.float32, torch.bfloat16)
    _check(lib.rllm_gemm_small_m(_ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out),
                                 c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(code), _stream()),
           "gemm_small_m")


def gemm_small_m_residual(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor,
                          w_next: Optional[torch.Tensor]):
    """h += x . w^T (h float32, in place) for M <= 16 rows of bfloat16.  Returns
    (parts, scaled): parts float32 [P, M], whose sum over P is each row's new sum of
    squares; scaled = bfloat16(h * w_next) [M, N] if the weight ``w_next`` of the norm
    that reads h next is given, else None."""
    lib = build.load_library("gemm_small_m")
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and w.shape[1] == K
    assert h.dtype is torch.float32 and h.shape == (M, N) and h.stride(1) == 1
    assert x.stride(1) == 1 and w.stride(1) == 1
    P = int(lib.rllm_gemm_small_m_parts(c_int(N)))
    parts = torch.empty((P, M), dtype=torch.float32, device=x.device)
    scaled = None
    if w_next is not None:
        assert w_next.numel() == N and w_next.is_contiguous() and w_next.dtype in (torch.float32, torch.bfloat16)
        scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _check(lib.rllm_gemm_small_m_residual(_ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(h),
                                          c_int(h.stride(0)), _ptr(parts), _ptr(w_next),
                                          c_int(1 if w_next is not None and w_next.dtype is torch.float32 else 0),
                                          _ptr(scaled), c_int(N), c_int(M), c_int(N), c_int(K), _stream()),
           "gemm_small_m_residual")
    return parts, scaled


def gemm_small_m_rstd(x: torch.Tensor, parts: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor,
                      epilogue: str = "store") -> None:
    """out = (x . w^T) with row m scaled by 1 / sqrt(sum(parts[:, m]) / K + eps): with
    x and parts from ``gemm_small_m_residual`` this is rmsnorm(h) . w^T.  Epilogues
    as in ``gemm_small_m`` (bfloat16 out)."""
    lib = build.load_library("gemm_small_m")
    M, K = x.shape
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and w.shape[1] == K and out.dtype is torch.bfloat16
    assert parts.dtype is torch.float32 and parts.is_contiguous() and parts.shape[1] == M
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if epilogue == "silu_mul":
        N, code = w.shape[0] // 2, 2
        assert w.shape[0] == 2 * N
    else:
        N, code = w.shape[0], 0
    assert out.shape == (M, N)
    _check(lib.rllm_gemm_small_m_rstd(_ptr(x), c_int(x.stride(0)), _ptr(parts), c_int(parts.shape[0]), c_float(eps),
                                      _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(M),
                                      c_int(N), c_int(K), c_int(code), _stream()), "gemm_small_m_rstd")


_one_wave_tiles = {}


def small_m_rows(num_rows: int, dtype: torch.dtype, weights=()) -> bool:
    """Whether a step of this many rows goes through the weight-streaming kernels.  Up to 8 rows: always.
    9 to 16 rows: if every one of ``weights`` has few enough rows for the kernels' one-wave form (16 rows a
    CTA, seven CTAs an SM); measured at batch 16, context 4096, four layers: Llama-1B shapes 16 % faster
    than the library path, 3B shapes equal, 8B shapes (whose gate_up has too many rows) 6 % slower."""
    import os
    if dtype is not torch.bfloat16 or num_rows <= 0 or os.environ.get("RLLM_GEMM") == "library":
        return False
    if num_rows > int(os.environ.get("RLLM_FUSED_M_MAX", FUSED_M_MAX)):
        return False
    if num_rows <= SMALL_M_MAX:
        return True
    for w in weights:
        cap = _one_wave_tiles.get(w.device)
        if cap is None:
            cap = _one_wave_tiles[w.device] = 7 * torch.cuda.get_device_properties(w.device).multi_processor_count
        if w.shape[0] // 16 > cap:
            return False
    return True


def small_m_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    import os
    return (x.dtype is torch.bfloat16 and 0 < x.shape[0] <= SMALL_M_MAX and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and os.environ.get("RLLM_GEMM") != "library")


_gemm_err = {}


def gemm_error_word(device: torch.device) -> torch.Tensor:
    """The per-device error word of the tcgen05 GEMM (bit 4: a bounded wait ran out)."""
    t = _gemm_err.get(device)
    if t is None:
        t = _gemm_err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def check_gemm_errors(device: torch.device) -> None:
    t = _gemm_err.get(device)
    code = int(t.item()) if t is not None else 0
    if code:
        t.zero_()
        what = []
        if code & 16:
            what.append("gemm_tcgen05: a wait on an mbarrier ran out")
        raise KernelError("; ".join(what or [f"error word {code}"]) + "; the result of that product is undefined")


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: str = "store") -> None:
    """out = x . w^T for bfloat16 on the tcgen05 tensor cores (TMA in, TMEM accumulators).
    epilogue "store": out [M, N] bfloat16 or float32.  "silu_mul": w = [gate rows;
    up rows] stacked (2 N rows), out [M, N] bfloat16 = silu(x gate^T) * (x up^T)."""
    lib = build.load_library("gemm_tcgen05")
    M, K = x.shape
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if epilogue == "silu_mul":
        N = w.shape[0] // 2
        assert out.dtype is torch.bfloat16 and out.shape == (M, N) and w.shape[0] == 2 * N
        code = 2
    else:
        N = w.shape[0]
        assert out.shape == (M, N) and out.dtype in (torch.float32, torch.bfloat16)
        code = 1 if out.dtype is torch.float32 else 0
    _check(lib.rllm_gemm_tcgen05(_ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out),
                                 c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(code),
                                 _ptr(gemm_error_word(x.device)), _stream()), "gemm_tcgen05")


TCGEN05_MIN_TILES = 96    # below this many 128 x 256 output tiles the GPU is not filled: the library's
                          # small-tile kernels read the weight faster


def tcgen05_takes(x: torch.Tensor, w: torch.Tensor, silu: bool = False) -> bool:
    """Whether the tcgen05 kernel should compute x . w^T.  ``silu``: w is [gate; up] stacked and the
    output has half of w's rows.  With the environment variable RLLM_GEMM=tcgen05 every shape it can
    take goes to it (used by tests, so that tiny models run through it)."""
    import os
    mode = os.environ.get("RLLM_GEMM", "")
    if mode in ("library", "no_tcgen05"):
        return False
    ok = (x.dtype is torch.bfloat16 and x.shape[0] > 0 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
          and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
    if not ok or mode == "tcgen05":
        return ok
    n_out = w.shape[0] // 2 if silu else w.shape[0]
    tiles = -(-x.shape[0] // 128) * -(-n_out // (128 if silu else 256))
    return tiles >= TCGEN05_MIN_TILES


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """x . w^T through this engine's own bfloat16 kernels, or None if none of them
    takes the shape (the caller then uses the library's matrix product).  Few rows:
    the weight-streaming kernel; more: the tcgen05 kernel."""
    if small_m_takes(x, w):
        import os
        if w.shape[0] > 65536 and (x.shape[0] > 8 or os.environ.get("RLLM_HEAD") == "library"):
            return None                 # very tall weights (the vocabulary) at 9 to 16 rows: the library's kernel is ahead
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
        gemm_small_m(x, w, out)
        return out
    if tcgen05_takes(x, w):
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
        gemm_tcgen05(x, w, out)
        return out
    return None


# ---------------------------------------------------------------------------
def draw_normal(out: torch.Tensor, key: int, std: float, one_plus: bool = False) -> None:
    """Fills ``out`` (float32 or bfloat16, contiguous) with std * z or 1 + std * z, z the standard normals
    of the counter-based stream ``key``: element i is the same value wherever it is drawn
    (``rllm_b200.weights.counter_rng`` is the CPU twin)."""
    lib = build.load_library("weights_rng")
    _contig(out, "out")
    _check(lib.rllm_draw_normal(_ptr(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()),
                                ctypes.c_ulonglong(key & 0xFFFFFFFFFFFFFFFF), ctypes.c_double(std),
                                c_int(1 if one_plus else 0), _stream()), "draw_normal")


def draw_randint(out: torch.Tensor, key: int, high: int) -> None:
    """Fills ``out`` (int32, contiguous) with word i of the stream ``key`` modulo ``high``."""
    lib = build.load_library("weights_rng")
    assert out.dtype is torch.int32 and 0 < high < (1 << 32)
    _contig(out, "out")
    _check(lib.rllm_draw_randint(_ptr(out), c_longlong(out.numel()), ctypes.c_ulonglong(key & 0xFFFFFFFFFFFFFFFF),
                                 ctypes.c_uint(high), _stream()), "draw_randint")


# ---------------------------------------------------------------------------
_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = lowest index of the largest value of row r (float32 rows)."""
    lib = build.load_library("sampling")
    R, V = logits.shape
    assert logits.dtype is torch.float32 and out.dtype is torch.int32 and logits.stride(1) == 1
    split = int(lib.rllm_argmax_split(c_int(V)))
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch[1].numel() < R:
        rows = max(R, 256)
        scratch = (torch.empty(rows * 64 * 2, dtype=torch.int32, device=logits.device),
                   torch.zeros(rows, dtype=torch.int32, device=logits.device))
        _argmax_scratch[logits.device] = scratch
    _check(lib.rllm_argmax(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)), _ptr(out),
                           _ptr(scratch[0]), _ptr(scratch[1]), _stream()), "argmax")


def _sample_asserts(logits, temperature, top_k, top_p, min_p, seeds, gen_index, out):
    assert logits.dtype is torch.float32 and logits.stride(1) == 1
    assert temperature.dtype is torch.float32 and top_k.dtype is torch.int32
    assert top_p.dtype is torch.float32 and min_p.dtype is torch.float32
    assert seeds.dtype is torch.int64 and gen_index.dtype is torch.int64 and out.dtype is torch.int32


_sample_scratch = {}


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seeds: torch.Tensor, gen_index: torch.Tensor, out: torch.Tensor,
           with_select: bool = True) -> None:
    """out[r] = the next token of row r: argmax for greedy rows, else a draw after temperature, top-k,
    top-p and min-p.  Every row is worked on by several CTAs, in a chain of small kernels.
    ``with_select=False`` leaves the top-k / top-p kernels out (the caller knows that no row uses them)."""
    lib = build.load_library("sampling")
    R, V = logits.shape
    _sample_asserts(logits, temperature, top_k, top_p, min_p, seeds, gen_index, out)
    lib.rllm_sample_scratch_bytes.restype = c_longlong
    need = int(lib.rllm_sample_scratch_bytes(c_int(R), c_int(V)))
    scratch = _sample_scratch.get(logits.device)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=logits.device)
        _sample_scratch[logits.device] = scratch
    _check(lib.rllm_sample(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)), _ptr(temperature),
                           _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(seeds), _ptr(gen_index), _ptr(out),
                           _ptr(scratch), c_int(1 if with_select else 0), _stream()), "sample")


def sample_one_cta(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                   min_p: torch.Tensor, seeds: torch.Tensor, gen_index: torch.Tensor, out: torch.Tensor) -> None:
    """The same sampling with one CTA a row in one kernel (slow for large vocabularies; kept as the
    simple form that the chain of kernels is checked against)."""
    lib = build.load_library("sampling")
    R, V = logits.shape
    _sample_asserts(logits, temperature, top_k, top_p, min_p, seeds, gen_index, out)
    _check(lib.rllm_sample_one_cta(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)), _ptr(temperature),
                                   _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(seeds), _ptr(gen_index),
                                   _ptr(out), _stream()), "sample_one_cta")


def logit_edits(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, counts: torch.Tensor,
                bias: torch.Tensor, rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    lib = build.load_library("sampling")
    R, V = logits.shape
    _check(lib.rllm_logit_edits(_ptr(logits), c_int(V), c_int(logits.stride(0)), c_int(rows.numel()),
                                _ptr(rows), _ptr(tokens), _ptr(counts), _ptr(bias), _ptr(rep),
                                _ptr(freq), _ptr(pres), _stream()), "logit_edits")


def logit_mask(logits: torch.Tensor, allowed_start: Optional[torch.Tensor],
               allowed: Optional[torch.Tensor], sup_rows: Optional[torch.Tensor],
               sup_tokens: Optional[torch.Tensor]) -> None:
    lib = build.load_library("sampling")
    R, V = logits.shape
    n = 0 if sup_rows is None else sup_rows.numel()
    _check(lib.rllm_logit_mask(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)),
                               _ptr(allowed_start), _ptr(allowed), c_int(n), _ptr(sup_rows),
                               _ptr(sup_tokens), _stream()), "logit_mask")


def attention_prefill_bf16(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor,
                           vcache: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                           seq_lens: torch.Tensor, seq_begin: int, seq_end: int, num_tokens: int, nq: int,
                           nkv: int, d: int, window: int, scale: float, err: torch.Tensor) -> None:
    """Tensor-core attention of the prompt portions of sequences seq_begin .. seq_end-1."""
    lib = build.load_library("attention_mma")
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert q.dtype is torch.bfloat16 and kcache.dtype is torch.bfloat16 and out.dtype is torch.bfloat16
    _check(lib.rllm_attention_prefill_bf16(_ptr(q), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache),
                                           _ptr(block_table), c_int(block_table.shape[1]), _ptr(q_start),
                                           _ptr(seq_lens), c_int(seq_begin), c_int(seq_end), c_int(num_tokens),
                                           c_int(nq), c_int(nkv), c_int(d), c_int(kcache.shape[2]),
                                           c_int(kcache.shape[0]), c_int(window), c_float(scale), _ptr(err),
                                           _stream()), "attention_prefill_bf16")


def attention_prefill_tcgen05_supported(nq: int, nkv: int, d: int, page_size: int) -> bool:
    """The sizes the tcgen05 prompt attention takes: head size 64 or 128, pages of 16 keys up to a key
    tile (128 keys for head size 64, 64 for 128), up to 128 query heads per kv head."""
    g = nq // nkv if nkv else 0
    return (d in (64, 128) and page_size in (16, 32, 64, 128) and page_size <= 8192 // d
            and 1 <= g <= 128 and nq % nkv == 0)


def attention_prefill_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor,
                              vcache: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                              seq_lens: torch.Tensor, seq_begin: int, seq_end: int, num_tokens: int, nq: int,
                              nkv: int, d: int, window: int, scale: float, err: torch.Tensor) -> None:
    """Attention of the prompt portions of sequences seq_begin .. seq_end-1 on the
    tcgen05 tensor cores (same contract as ``attention_prefill_bf16``; ``q`` is the
    first of ``q.shape[0]`` rows of ``q_stride`` elements)."""
    lib = build.load_library("attention_tcgen05")
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert q.dtype is torch.bfloat16 and kcache.dtype is torch.bfloat16 and out.dtype is torch.bfloat16
    _check(lib.rllm_attention_prefill_tcgen05(_ptr(q), c_int(q_stride), c_int(q.shape[0]), _ptr(out), _ptr(kcache),
                                              _ptr(vcache), _ptr(block_table), c_int(block_table.shape[1]),
                                              _ptr(q_start), _ptr(seq_lens), c_int(seq_begin), c_int(seq_end),
                                              c_int(num_tokens), c_int(nq), c_int(nkv), c_int(d),
                                              c_int(kcache.shape[2]), c_int(kcache.shape[0]), c_int(window),
                                              c_float(scale), _ptr(err), _stream()), "attention_prefill_tcgen05")


_decode_counters = {}
_retired_counters = []          # buffers that grew out of use: captured graphs may still hold their address


def _counters_for(device: torch.device, n: int) -> torch.Tensor:
    """Zeroed per-device counters of the decode kernel's split merge; the kernel
    leaves them zero, so one buffer serves every call (also under CUDA graphs).
    A buffer that is outgrown is never freed (a captured graph replays with its
    address), and none is made while a stream is being captured."""
    buf = _decode_counters.get(device)
    if buf is None or buf.numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"attention_decode: {n} merge counters are needed and the buffer cannot grow during "
                              "a stream capture; run this size once outside a capture first")
        if buf is not None:
            _retired_counters.append(buf)
        buf = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _decode_counters[device] = buf
    return buf


def attention_decode_bf16(qkv: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor,
                          vcache: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                          num_seqs: int, max_seq_len: int, nq: int, nkv: int, d: int, window: int,
                          scale: float, err: torch.Tensor, workspace: Optional[torch.Tensor] = None,
                          inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0,
                          write_kv: bool = False) -> None:
    """Split-KV tensor-core attention of sequences 0 .. num_seqs-1, one query token
    each: row s of ``qkv`` holds the token's q heads (and behind them its k and v
    heads if ``write_kv``), row s of ``out`` gets the result.  ``rotary_dim`` > 0
    rotates q (and the new k) in the kernel; ``write_kv`` stores the token's k and
    v into the cache in the kernel.  ``max_seq_len`` bounds every length.  The
    workspace (float32, ``attention_decode_workspace`` elements) holds the splits'
    partial results; it is allocated here if not given."""
    lib = build.load_library("attention_mma")
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert qkv.dtype is torch.bfloat16 and kcache.dtype is torch.bfloat16 and out.dtype is torch.bfloat16
    need = attention_decode_workspace(num_seqs, nq, d, max_seq_len)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.float32, device=qkv.device)
    assert workspace.dtype is torch.float32 and workspace.numel() >= need
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype is torch.float64 and inv_freq.numel() == rotary_dim // 2
    counters = _counters_for(qkv.device, num_seqs * nkv)
    _check(lib.rllm_attention_decode_bf16(_ptr(qkv), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache),
                                          _ptr(block_table), c_int(block_table.shape[1]), _ptr(seq_lens),
                                          c_int(num_seqs), c_int(max_seq_len), c_int(nq), c_int(nkv), c_int(d),
                                          c_int(kcache.shape[2]), c_int(kcache.shape[0]), c_int(window),
                                          c_float(scale), _ptr(inv_freq), c_int(rotary_dim),
                                          c_int(1 if write_kv else 0), _ptr(workspace), _ptr(counters),
                                          _ptr(err), _stream()), "attention_decode_bf16")


def attention_decode_workspace(num_seqs: int, nq: int, d: int, max_seq_len: int) -> int:
    lib = build.load_library("attention_mma")
    lib.rllm_attention_decode_workspace.restype = c_longlong
    return int(lib.rllm_attention_decode_workspace(c_int(num_seqs), c_int(nq), c_int(d), c_int(max_seq_len)))


def mma_attention_takes(nq: int, nkv: int, d: int) -> bool:
    return d in (16, 32, 64, 128) and nq % nkv == 0 and nq // nkv <= 16


def use_mma_attention(dtype: torch.dtype, nq: int, nkv: int, d: int) -> bool:
    """bfloat16 with a head size the tensor-core attention kernels take; other
    cases (float32, other head sizes) go to the CUDA-core kernel."""
    import os
    return dtype is torch.bfloat16 and mma_attention_takes(nq, nkv, d) and os.environ.get("RLLM_ATTENTION") != "simt"


def use_tcgen05_attention(dtype: torch.dtype, nq: int, nkv: int, d: int, page_size: int) -> bool:
    """Prompt portions go to the tcgen05 attention kernel when it takes the sizes;
    RLLM_ATTENTION=mma (or simt) keeps them on the older kernels."""
    import os
    return (dtype is torch.bfloat16 and attention_prefill_tcgen05_supported(nq, nkv, d, page_size)
            and os.environ.get("RLLM_ATTENTION") not in ("simt", "mma"))


def decode_advance(token_ids: torch.Tensor, positions: torch.Tensor, seq_lens: torch.Tensor,
                   sampled: torch.Tensor, history_row: Optional[torch.Tensor], count: Optional[int] = None) -> None:
    """For the first ``count`` rows (all by default): token_ids = sampled; positions += 1; seq_lens += 1;
    history_row = sampled.  ``history_row`` may be pinned host memory: the kernel then writes the tokens
    where the host reads them, and no copy stands in the stream."""
    lib = build.load_library("elementwise")
    n = token_ids.numel() if count is None else int(count)
    assert n <= token_ids.numel() and n <= sampled.numel() and (history_row is None or n <= history_row.numel())
    if history_row is not None and not history_row.is_cuda:
        # page-locked host memory has the same address on the device
        if not history_row.is_pinned() or history_row.dtype is not torch.int32:
            raise KernelError("decode_advance: a host row must be pinned int32 memory")
        row = c_void_p(history_row.data_ptr())
    else:
        row = _ptr(history_row)
    _check(lib.rllm_decode_advance(_ptr(token_ids), _ptr(positions), _ptr(seq_lens), _ptr(sampled),
                                   row, c_int(n), _stream()), "decode_advance")


def logprobs(logits: torch.Tensor, tokens: torch.Tensor, top_n: int):
    """Natural-log probabilities from raw logits float32 [R, V]: (lp [R] of ``tokens`` int32 [R], ids int32
    [R, top_n] and values float32 [R, top_n] of every row's ``top_n`` likeliest tokens, descending, the lower
    index first among equals; id -1 where nothing is left)."""
    lib = build.load_library("sampling")
    R, V = logits.shape
    assert logits.dtype is torch.float32 and logits.stride(1) == 1 and tokens.dtype is torch.int32 and tokens.numel() == R
    lp = torch.empty(R, dtype=torch.float32, device=logits.device)
    ids = torch.empty((R, top_n), dtype=torch.int32, device=logits.device)
    vals = torch.empty((R, top_n), dtype=torch.float32, device=logits.device)
    _check(lib.rllm_logprobs(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)), _ptr(tokens), c_int(top_n),
                             _ptr(lp), _ptr(ids) if top_n else c_void_p(0), _ptr(vals) if top_n else c_void_p(0),
                             _stream()), "logprobs")
    return lp, ids, vals
