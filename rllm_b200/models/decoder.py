"""The generic decoder: any ``ModelSpec`` built from registered parts.

This is the only model class of the framework.  An architecture is a function
from its typed configuration to a ``ModelSpec``; the decoder builds the parts
the spec names, collects the tensors they declare, works out which runs of the
order need which kind of cache, and runs a step:

    embedding -> for each run of the order: block(run.layer) with the cache of
    run.cache -> final norm on the rows that were asked for -> head.

(The reference's forward is the fixed loop of crates/rllm-model/src/llama.rs:283-326,
with the head applied to every row at :70.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts import registry as part_registry
from ..parts.base import KVCacheView, StateCacheView, StepContext
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.spec import KVPagesNeed, ModelSpec, StateNeed, TensorSpec
from ..weights.loader import WeightSource, load_tensors


@dataclass
class CacheLayout:
    """groups[g]: the need shared by the runs of group g.  owners[g]: the runs
    (indices into the order) that own storage in group g.  run_group[i] and
    run_owner[i]: the group of run i and the run whose storage it uses (None:
    the run's mixer keeps nothing)."""

    groups: List[object]
    owners: List[List[int]]
    run_group: List[Optional[int]]
    run_owner: List[Optional[int]]


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = TokenEmbedding(spec.embedding)
        self.blocks = []
        for ls in spec.layers:
            mixer = part_registry.build_part("mixer", ls.mixer, prefix=ls.prefix + _sub(ls.mixer))
            ffn = part_registry.build_part("feed_forward", ls.ffn, prefix=ls.prefix + _sub(ls.ffn))
            norms = [part_registry.build_part("norm", n, prefix=ls.prefix) for n in ls.norms]
            if ls.block not in part_registry.BLOCKS:
                raise KeyError(f"no block arrangement {ls.block!r}; known: {sorted(part_registry.BLOCKS)}")
            self.blocks.append(part_registry.BLOCKS[ls.block](mixer, ffn, norms))
        self.final_norm = part_registry.build_part("norm", spec.final_norm)
        self.head = OutputHead(spec.head)
        self.layout = self._cache_layout()
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # -- weights ----------------------------------------------------------
    def parts(self):
        out = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        out += [self.final_norm, self.head]
        return out

    def tensor_specs(self) -> List[TensorSpec]:
        seen: Dict[str, TensorSpec] = {}
        for part in self.parts():
            for ts in part.tensor_specs():
                if ts.name in seen and seen[ts.name].shape != ts.shape:
                    raise ValueError(f"tensor {ts.name!r} is declared twice with different shapes")
                seen.setdefault(ts.name, ts)
        return list(seen.values())

    def load(self, source: WeightSource, run_dtype: torch.dtype, device: torch.device) -> None:
        ignored = [n for part in self.parts() for n in part.ignored_tensors()]
        tensors = load_tensors(self.tensor_specs(), source, run_dtype, device, ignored)
        for part in self.parts():
            part.load(tensors)
        self.dtype, self.device = run_dtype, device

    def num_weight_bytes(self) -> int:
        seen, total = set(), 0
        for part in self.parts():
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    # -- cache ------------------------------------------------------------
    def _cache_layout(self) -> CacheLayout:
        groups: List[object] = []
        owners: List[List[int]] = []
        run_group: List[Optional[int]] = []
        run_owner: List[Optional[int]] = []
        for i, run in enumerate(self.spec.order):
            need = self.blocks[run.layer].mixer.cache_need()
            if need is None:
                run_group.append(None)
                run_owner.append(None)
                continue
            owner_need = self.blocks[self.spec.order[run.cache].layer].mixer.cache_need()
            if run.cache != i and owner_need != need:
                raise ValueError(f"order[{i}] reads the cache of run {run.cache}, whose mixer keeps "
                                 f"{owner_need}, not {need}")
            if need not in groups:
                groups.append(need)
                owners.append([])
            g = groups.index(need)
            if run.cache == i:
                owners[g].append(i)
            run_group.append(g)
            run_owner.append(run.cache)
        return CacheLayout(groups, owners, run_group, run_owner)

    # -- compute ----------------------------------------------------------
    def forward(self, token_ids: torch.Tensor, ctx: StepContext, logit_rows: torch.Tensor,
                storage) -> torch.Tensor:
        """Logits float32 [R, vocab] at the rows ``logit_rows`` (int32 indices
        into this step's tokens).  ``storage.view(run_index)`` gives a run's
        cache view."""
        h = self.embedding.forward(token_ids, ctx.err)
        pending = None
        order = self.spec.order
        for i, run in enumerate(order):
            block = self.blocks[run.layer]
            if getattr(block, "takes_next_norm", False) and i + 1 < len(order):
                # the norm that reads the stream after this block: the block may prepare its input
                nxt = getattr(self.blocks[order[i + 1].layer], "norms", None)
                h, pending = block.forward(h, pending, ctx, storage.view(i), next_norm=nxt[0] if nxt else None)
            else:
                h, pending = block.forward(h, pending, ctx, storage.view(i))
        if logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        if not isinstance(pending, torch.Tensor):
            pending = None                      # a block that adds into the stream itself left it complete
        xn = self.final_norm.gather_forward(h, pending, logit_rows, ctx.act_dtype)
        return self.head.forward(xn)


def _sub(part_spec) -> str:
    """Tensor-name segment between the layer prefix and a part's tensors: the spec's
    ``tensor_prefix`` (none: the part's tensors lie directly under the layer prefix)."""
    sub = part_spec.get().get("tensor_prefix")
    return "" if sub is None else str(sub)
