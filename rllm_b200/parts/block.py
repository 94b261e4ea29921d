"""Arrangements of a mixer, a feed-forward and norms in a layer.

``pre_norm`` is the Llama decoder layer
(crates/rllm-model/src/layers.rs:677-699):
    h   = x + mixer(norm_0(x))
    out = h + ffn(norm_1(h))
The residual stream h is float32 and every add into it is a float32 add.  The
last add of a block is not done here: the block returns (h, pending) with
out = h + pending, and whichever norm reads the stream next adds ``pending``
in the same kernel that normalises.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .base import FeedForward, Mixer, Norm, StepContext
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock:
    def __init__(self, mixer: Mixer, ffn: FeedForward, norms: List[Norm]):
        if len(norms) != 2:
            raise ValueError("a pre_norm block has two norms: before the mixer and before the feed-forward")
        self.mixer, self.ffn, self.norms = mixer, ffn, norms

    def parts(self):
        return [self.norms[0], self.mixer, self.norms[1], self.ffn]

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache) -> Tuple[torch.Tensor, torch.Tensor]:
        if pending is None:
            xn = self.norms[0].forward(h, ctx.act_dtype)
        else:
            xn = self.norms[0].add_forward(h, pending)
        a = self.mixer.forward(xn, ctx, cache)
        xn = self.norms[1].add_forward(h, a)
        return h, self.ffn.forward(xn)
