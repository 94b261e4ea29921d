"""SiLU-gated feed-forward: down(silu(gate(x)) * up(x)), no bias
(crates/rllm-model/src/layers.rs:214-220).  gate and up are one matrix product
over the stacked weights [Wgate; Wup]; silu(z) = z / (1 + exp(-z)) and the
product with up are computed in float32.

params: hidden_size, intermediate_size, tensor_names (the names of the three
weights below the part's prefix, keys "gate", "up", "down").
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward
from .base import ScaledRows
from .linear import fused_residual_takes, linear
from .registry import register_part
from .spec import PartSpec, TensorSpec


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        names = dict(spec.get().get("tensor_names") or ())
        if sorted(names) != ["down", "gate", "up"]:
            raise ValueError("a gated_mlp spec names its weights: tensor_names with the keys gate, up, down")
        self.names = {k: str(v) for k, v in names.items()}
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def _names(self):
        p = self.prefix
        return tuple(p + self.names[k] for k in ("gate", "up", "down"))

    def tensor_specs(self) -> List[TensorSpec]:
        g, u, d = self._names()
        return [TensorSpec(g, (self.inter, self.hidden)), TensorSpec(u, (self.inter, self.hidden)),
                TensorSpec(d, (self.hidden, self.inter))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u, d = self._names()
        self.w_gate_up = torch.cat([tensors[g], tensors[u]], dim=0).contiguous()
        self.w_down = tensors[d]

    def fused_residual(self, num_rows: int, dtype: torch.dtype) -> bool:
        return fused_residual_takes(num_rows, dtype, self.w_gate_up, self.w_down)

    def forward(self, x, residual=None):
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        if isinstance(x, ScaledRows):
            # the rows' 1 / rms is applied to gate and up before the SiLU
            ops.gemm_small_m_rstd(x.x, x.parts, x.eps, self.w_gate_up, act, "silu_mul")
        elif ops.small_m_takes(x, self.w_gate_up):
            # few rows: one kernel streams [Wgate; Wup] once and applies silu(gate) * up to its accumulators
            ops.gemm_small_m(x, self.w_gate_up, act, "silu_mul")
        elif ops.tcgen05_takes(x, self.w_gate_up, silu=True):
            # many rows: tensor-core tiles of 128 gate and 128 up features, silu(gate) * up in the epilogue
            ops.gemm_tcgen05(x, self.w_gate_up, act, "silu_mul")
        else:
            gate_up = linear(x, self.w_gate_up)                   # [T, 2I]
            ops.silu_mul(gate_up, act)
        return linear(act, self.w_down, residual=residual)
