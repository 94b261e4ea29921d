"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, eps inside the root, the weight
as it is, all in float32 (crates/rllm-model/src/layers.rs:133-140).  ``eps``
is a parameter (the reference hard-codes 1e-6, crates/rllm-model/src/llama.rs:183).

The norm reads the float32 residual stream; ``add_forward`` first adds a
block's output to it in float32, in the same kernel.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Norm, RowSumsq, ScaledRows
from .registry import register_part
from .spec import PartSpec, TensorSpec


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, name (tensor name below the prefix)."""
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.name = prefix + str(spec["name"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.size,), role="vector", init=("one_plus_normal", 0.1))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def forward(self, x: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=act_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out)
        return out

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=delta.dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, writeback=True)
        return out

    def scaled_input(self, stats: RowSumsq) -> Optional[ScaledRows]:
        """The normalised stream for a product that applies the rows' factors itself, if
        ``stats`` was prepared with this norm's weight."""
        if stats.scaled is None or stats.scaled_by is not self.weight:
            return None
        return ScaledRows(stats.scaled, stats.parts, self.eps)

    def gather_forward(self, x, delta, rows, act_dtype):
        out = torch.empty((rows.numel(), x.shape[1]), dtype=act_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows)
        return out
