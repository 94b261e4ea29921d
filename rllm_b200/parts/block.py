"""Arrangements of a mixer, a feed-forward and norms in a layer.

``pre_norm`` is the Llama decoder layer
(crates/rllm-model/src/layers.rs:677-699):
    h   = x + mixer(norm_0(x))
    out = h + ffn(norm_1(h))
The residual stream h is float32 and every add into it is a float32 add.  The
last add of a block is not done here: the block returns (h, pending) with
out = h + pending, and whichever norm reads the stream next adds ``pending``
in the same kernel that normalises.

With few rows (decoding) and parts that can do it, no norm kernel runs at all:
the product that ends the mixer (and the feed-forward) adds into h itself and
leaves what the next norm needs, and the product that follows the norm applies
it (see ``RowSumsq`` and ``ScaledRows`` in ``parts/base.py``).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .base import FeedForward, Mixer, Norm, RowSumsq, StepContext
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock:
    def __init__(self, mixer: Mixer, ffn: FeedForward, norms: List[Norm]):
        if len(norms) != 2:
            raise ValueError("a pre_norm block has two norms: before the mixer and before the feed-forward")
        self.mixer, self.ffn, self.norms = mixer, ffn, norms

    def parts(self):
        return [self.norms[0], self.mixer, self.norms[1], self.ffn]

    takes_next_norm = True

    def _fused(self, num_rows: int, ctx: StepContext) -> bool:
        import os
        return (all(getattr(p, "fused_residual", None) is not None and p.fused_residual(num_rows, ctx.act_dtype)
                    for p in (self.mixer, self.ffn))
                and all(hasattr(n, "scaled_input") for n in self.norms)
                and os.environ.get("RLLM_FUSED_NORM") != "0")

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, cache, next_norm=None):
        """``next_norm``: the norm that reads the stream after this block, if the caller knows it."""
        if self._fused(h.shape[0], ctx):
            xn = self.norms[0].scaled_input(pending) if isinstance(pending, RowSumsq) else None
            if xn is None:
                if pending is None or isinstance(pending, RowSumsq):
                    xn = self.norms[0].forward(h, ctx.act_dtype)
                else:
                    xn = self.norms[0].add_forward(h, pending)
            stats = self.mixer.forward(xn, ctx, cache, residual=(h, self.norms[1]))
            stats = self.ffn.forward(self.norms[1].scaled_input(stats), residual=(h, next_norm))
            return h, stats
        if isinstance(pending, RowSumsq):
            pending = None                      # h is complete
        if pending is None:
            xn = self.norms[0].forward(h, ctx.act_dtype)
        else:
            xn = self.norms[0].add_forward(h, pending)
        a = self.mixer.forward(xn, ctx, cache)
        xn = self.norms[1].add_forward(h, a)
        return h, self.ffn.forward(xn)
