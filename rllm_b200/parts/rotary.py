"""Rotary position encoding, rotate-half convention
(crates/rllm-model/src/rope.rs:57-82), with the frequency table
f_i = theta^(-2i/d) (rope.rs:13-15) built in float64 on the host and, if
asked, rescaled by the llama3 rule: by wavelength 2*pi/f_i, shorter than
orig/high_freq_factor: kept; longer than orig/low_freq_factor: divided by
``factor``; between: blended linearly in orig/wavelength.  (The reference
declares the scaling struct, crates/rllm-core/src/config.rs:25-31, and never
fills it, crates/rllm-model/src/hf_config.rs:68.)

No table over positions is stored: the kernel computes cos and sin of
position * f_i in float64 per token, which is what the reference's table holds
(rope.rs:24-28), for any position.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from ..kernels import ops
from .base import PositionEncoding
from .registry import register_part
from .spec import PartSpec


def rotary_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> List[float]:
    freqs = [1.0 / (float(theta) ** (i / rotary_dim)) for i in range(0, rotary_dim, 2)]
    if not scaling:
        return freqs
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < orig / high:
            out.append(f)
        elif wavelength > orig / low:
            out.append(f / factor)
        else:
            s = (orig / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


@register_part("position_encoding", "rotary")
class Rotary(PositionEncoding):
    """params: head_dim, rotary_dim (<= head_dim, even), theta, scaling (dict or None),
    ignored_tensors (names below the mixer's prefix under which checkpoints of the family store
    a frequency table; it is computed here, so such a tensor is passed over)."""
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.head_dim = int(p["head_dim"])
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        scaling = p.get("scaling")
        self.scaling = dict(scaling) if scaling else None
        self.freqs = rotary_frequencies(self.rotary_dim, float(p["theta"]), self.scaling)
        self._table: Optional[torch.Tensor] = None
        self._ignored = [prefix + str(n) for n in (p.get("ignored_tensors") or ())]

    def ignored_tensors(self) -> List[str]:
        return list(self._ignored)

    def load(self, tensors) -> None:
        pass

    def table(self, device) -> torch.Tensor:
        if self._table is None or self._table.device != device:
            self._table = torch.tensor(self.freqs, dtype=torch.float64, device=device)
        return self._table

    def fused_rotary(self, device=None) -> Optional[Tuple[torch.Tensor, int]]:
        return self.table(device), self.rotary_dim


@register_part("position_encoding", "none")
class NoPosition(PositionEncoding):
    graph_safe = True

    def fused_rotary(self, device=None):
        return None, 0
