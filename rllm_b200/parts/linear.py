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


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
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
