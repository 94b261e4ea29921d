"""y = x . W^T with W stored [out, in], no bias
(crates/rllm-model/src/layers.rs:162-175).

float32: the engine's own FFMA kernel (no tensor cores, no reduced-precision
matrix mode).  bfloat16: the engine's tensor-core kernels where they take the
shape, else the vendor library's matrix product, which is where the reference
calls a library too (Candle's matmul at layers.rs:170).  Accumulation is
float32 in every case; ``out_dtype=torch.float32`` keeps the accumulator
unrounded (used for the logits).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import RowSumsq, ScaledRows


def fused_residual_takes(num_rows: int, dtype: torch.dtype, *weights: torch.Tensor) -> bool:
    """Whether ``linear`` takes a ``ScaledRows`` input and a ``residual`` for these weights and rows."""
    return ops.small_m_rows(num_rows, dtype, weights) and all(
        w.dtype is torch.bfloat16 and w.shape[1] % 8 == 0 and w.stride(0) % 8 == 0 and w.stride(1) == 1 for w in weights)


def linear(x, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None, residual=None):
    """``residual=(h, norm)``: the product is added into h (float32, in place) and a ``RowSumsq`` is
    returned; ``x`` may be a ``ScaledRows``.  Both only where ``fused_residual_takes`` says so."""
    if isinstance(x, ScaledRows):
        assert residual is None and fused_residual_takes(x.shape[0], x.dtype, weight)
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        ops.gemm_small_m_rstd(x.x, x.parts, x.eps, weight, out)
        return out
    if residual is not None:
        h, norm = residual
        assert fused_residual_takes(x.shape[0], x.dtype, weight)
        w_next = getattr(norm, "weight", None) if norm is not None and hasattr(norm, "scaled_input") else None
        parts, scaled = ops.gemm_small_m_residual(x, weight, h, w_next)
        return RowSumsq(parts, scaled, w_next)
    assert x.dim() == 2 and weight.dim() == 2 and x.shape[1] == weight.shape[1], (x.shape, weight.shape)
    if not x.is_cuda:
        raise ops.KernelError("linear: CUDA tensors only; the engine has no CPU path")
    M, N = x.shape[0], weight.shape[0]
    out_dtype = out_dtype or x.dtype
    if x.dtype is torch.float32:
        assert weight.dtype is torch.float32 and out_dtype is torch.float32
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        if M:
            ops.gemm_f32(x, weight, out)
        return out
    assert x.dtype is torch.bfloat16 and weight.dtype is torch.bfloat16
    if M == 0:
        return torch.empty((0, N), dtype=out_dtype, device=x.device)
    fast = ops.gemm_bf16(x, weight, out_dtype) if hasattr(ops, "gemm_bf16") else None
    if fast is not None:
        return fast
    if out_dtype is torch.float32:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    return torch.mm(x, weight.t())
