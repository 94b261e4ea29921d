"""Grouped-query causal attention over a paged cache: the Llama mixer.

q, k, v projections without bias (one fused matrix product over the stacked
weights), head split, position encoding on q and k, write of k and v into the
run's cache pages, attention of every query token over its sequence's cache
through the block table, output projection
(crates/rllm-model/src/layers.rs:280-347 for the math, :363-571 for the paged
intent).  kv head of query head h is h // (nq // nkv)
(crates/rllm-kernels/src/cuda/paged_attention.cu:113); scores are scaled by
1/sqrt(head_dim) (layers.rs:326-329) unless ``scale`` is given.

Portions of prompts and single decoded tokens are one code path: the tokens
of this step are written to the cache first and every query then reads keys
0 .. its own position (or its window) from the cache.

params: hidden_size, num_heads, num_kv_heads, head_dim, window (None: all
keys), scale (None: 1/sqrt(head_dim)), position (PartSpec), shares_kv (True:
the run reads another run's cache, has no k/v projections and writes nothing),
tensor_names (the names of the four projection weights below the part's prefix,
keys "q", "k", "v", "o": the architecture gives them, the part knows none).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import KVCacheView, Mixer, StepContext
from .linear import fused_residual_takes, linear
from .registry import build_part, register_part
from .spec import KVPagesNeed, PartSpec, TensorSpec


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    @property
    def graph_safe(self) -> bool:
        """forward launches kernels only; so a decode step can be captured if the position part's ``apply`` can."""
        return bool(self.position.graph_safe)

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.d)
        self.shares_kv = bool(p.get("shares_kv", False))
        if self.nq % self.nkv:
            raise ValueError(f"num_heads {self.nq} must be a multiple of num_kv_heads {self.nkv}")
        if self.d % 16 or self.d > 256:
            raise ValueError(f"head_dim {self.d}: the attention kernels take multiples of 16 up to 256")
        names = dict(p.get("tensor_names") or ())
        if sorted(names) != ["k", "o", "q", "v"]:
            raise ValueError("an attention spec names its weights: tensor_names with the keys q, k, v, o")
        self.names = {k: str(v) for k, v in names.items()}
        pos = p.get("position")
        self.position = build_part("position_encoding", pos if pos is not None else PartSpec.of("none"),
                                   prefix=prefix)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    # -- weights ----------------------------------------------------------
    def _names(self):
        p = self.prefix
        return tuple(p + self.names[k] for k in ("q", "k", "v", "o"))

    def ignored_tensors(self) -> List[str]:
        return self.position.ignored_tensors()

    def tensor_specs(self) -> List[TensorSpec]:
        q, k, v, o = self._names()
        specs = [TensorSpec(q, (self.nq * self.d, self.hidden))]
        if not self.shares_kv:
            specs += [TensorSpec(k, (self.nkv * self.d, self.hidden)),
                      TensorSpec(v, (self.nkv * self.d, self.hidden))]
        specs.append(TensorSpec(o, (self.hidden, self.nq * self.d)))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, k, v, o = self._names()
        if self.shares_kv:
            self.w_qkv = tensors[q]
        else:
            # stacked [Wq; Wk; Wv]: one matrix product gives a token's q, k and v side by side
            self.w_qkv = torch.cat([tensors[q], tensors[k], tensors[v]], dim=0).contiguous()
        self.w_o = tensors[o]

    def cache_need(self):
        return KVPagesNeed(self.nkv, self.d, self.window)

    # -- compute ----------------------------------------------------------
    def fused_residual(self, num_rows: int, dtype: torch.dtype) -> bool:
        return fused_residual_takes(num_rows, dtype, self.w_qkv, self.w_o)

    def forward(self, x, ctx: StepContext, cache: KVCacheView, residual=None):
        out = self.attend(linear(x, self.w_qkv), ctx, cache)          # qkv [T, (nq + 2 nkv) d]
        return linear(out, self.w_o, residual=residual)

    def attend(self, qkv: torch.Tensor, ctx: StepContext, cache: KVCacheView) -> torch.Tensor:
        """From the tokens' projections (q, k and v heads side by side) to the attention's output
        [T, nq * d], before the output projection: position encoding, cache write, attention."""
        x = qkv
        T = qkv.shape[0]
        nkv_here = 0 if self.shares_kv else self.nkv
        table = ctx.block_tables[cache.group]
        fused = self.position.fused_rotary(x.device)
        writes = cache.writes and not self.shares_kv
        if fused is None:
            q = qkv[:, : self.nq * self.d].view(T, self.nq, self.d)
            k = qkv[:, self.nq * self.d: (self.nq + nkv_here) * self.d].view(T, nkv_here, self.d) \
                if nkv_here else None
            self.position.apply(q, k, ctx.positions)
            fused = (None, 0)
        inv_freq, rd = fused
        out = torch.empty((T, self.nq * self.d), dtype=x.dtype, device=x.device)
        window = int(self.window or 0)
        stride = qkv.shape[1]
        use_mma = ops.use_mma_attention(x.dtype, self.nq, self.nkv, self.d)
        # sequences with one token: rotation, cache write and attention in one kernel
        nd = ctx.num_decode if use_mma else 0
        if nd:
            ops.attention_decode_bf16(qkv, stride, out, cache.k, cache.v, table, ctx.seq_lens, nd,
                                      max(ctx.seq_lens_host[:nd]), self.nq, self.nkv, self.d, window, self.scale,
                                      ctx.err, inv_freq=inv_freq, rotary_dim=rd, write_kv=writes)
        if T > nd:
            ops.rope_kv_write(qkv[nd:], ctx.positions[nd:], ctx.token_seq[nd:], inv_freq, rd, table, cache.k,
                              cache.v, self.nq, nkv_here, self.d, ctx.err, write_kv=writes)
            if ops.use_tcgen05_attention(x.dtype, self.nq, self.nkv, self.d, cache.k.shape[2]):
                ops.attention_prefill_tcgen05(qkv, stride, out, cache.k, cache.v, table, ctx.q_start, ctx.seq_lens,
                                              nd, ctx.num_seqs, T - nd, self.nq, self.nkv, self.d, window,
                                              self.scale, ctx.err)
            elif use_mma:
                ops.attention_prefill_bf16(qkv, stride, out, cache.k, cache.v, table, ctx.q_start, ctx.seq_lens,
                                           nd, ctx.num_seqs, T - nd, self.nq, self.nkv, self.d, window,
                                           self.scale, ctx.err)
            else:
                ops.attention_simt(qkv, stride, out, cache.k, cache.v, table, ctx.positions, ctx.token_seq,
                                   self.nq, self.nkv, self.d, window, self.scale, ctx.err)
        return out
