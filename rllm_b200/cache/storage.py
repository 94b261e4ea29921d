"""Device storage of the cache, laid out from what the model's runs declare.

Paged group: every run that owns a cache slot gets K and V tensors
[num_pages, num_kv_heads, page_size, head_dim] in the activation dtype.  A
page id indexes the same page in every run of the group, like the reference's
block ids index every layer's buffer (crates/rllm-cache/src/spec.rs:26-32).
Inside a page the tokens of one kv head are contiguous rows of head_dim, so a
(page, head) tile is one contiguous block (the reference's
[blocks, heads, head_dim, block_size], spec.rs:63-68, strides the hot axis).
State group: every owning run gets float32 [max_seqs, *shape], indexed by a
request's state slot.  All storage is allocated once, here.

Every paged buffer has one page more than the manager hands out: page
``spare_page(group)`` belongs to no request; every state buffer has one slot
more, ``spare_slot``.  The rows that pad a decode step to a captured batch size
read and write there.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..parts.base import KVCacheView, StateCacheView
from ..parts.spec import KVPagesNeed, StateNeed


def page_bytes(need: KVPagesNeed, page_size: int, elem_size: int) -> int:
    """Bytes of one page of one run: K and V."""
    return 2 * need.num_kv_heads * page_size * need.head_dim * elem_size


class CacheStorage:
    def __init__(self, layout, page_size: int, num_pages: Sequence[int], max_seqs: int,
                 dtype: torch.dtype, device: torch.device):
        self.layout = layout
        self.page_size = page_size
        self.kv: Dict[int, tuple] = {}
        self.state: Dict[int, torch.Tensor] = {}
        paged = [g for g, n in enumerate(layout.groups) if isinstance(n, KVPagesNeed)]
        pages_of = dict(zip(paged, num_pages))
        self._pages_of = pages_of
        self.spare_slot = max_seqs           # the state slot that no request ever holds
        for g, need in enumerate(layout.groups):
            for run in layout.owners[g]:
                if isinstance(need, KVPagesNeed):
                    shape = (pages_of[g] + 1, need.num_kv_heads, page_size, need.head_dim)
                    self.kv[run] = (torch.zeros(shape, dtype=dtype, device=device),
                                    torch.zeros(shape, dtype=dtype, device=device))
                elif isinstance(need, StateNeed):
                    self.state[run] = torch.zeros((max_seqs + 1,) + tuple(need.shape), dtype=torch.float32,
                                                  device=device)
                else:
                    raise TypeError(f"unknown cache need {need!r}")

    def spare_page(self, group: int) -> int:
        """The id of the page of this paged group that no request ever holds."""
        return self._pages_of[group]

    def view(self, run_index: int):
        g = self.layout.run_group[run_index]
        if g is None:
            return None
        owner = self.layout.run_owner[run_index]
        writes = owner == run_index
        if owner in self.kv:
            k, v = self.kv[owner]
            return KVCacheView(k, v, g, writes)
        return StateCacheView(self.state[owner], g, writes)

    def zero_slots(self, slots: List[int]) -> None:
        """Zero the state of newly handed-out slots."""
        if not slots or not self.state:
            return
        idx = torch.tensor(slots, dtype=torch.long, device=next(iter(self.state.values())).device)
        for t in self.state.values():
            t.index_fill_(0, idx, 0.0)

    def copy_for_fork(self, copies, slots) -> None:
        """The device side of ``CacheManager.fork``: every owning run of a group copies the
        page (K and V, one device-to-device copy each, on the current stream) and every
        state buffer copies the slot.  The reference has the copy kernel
        (crates/rllm-kernels/src/cuda/cache_ops.cu:252-279) and never calls it."""
        for g, src, dst in copies:
            for run in self.layout.owners[g]:
                k, v = self.kv[run]
                k[dst].copy_(k[src], non_blocking=True)
                v[dst].copy_(v[src], non_blocking=True)
        src, dst = slots
        for t in self.state.values():
            t[dst].copy_(t[src], non_blocking=True)

    def num_bytes(self) -> int:
        n = sum(k.numel() * k.element_size() * 2 for k, _ in self.kv.values())
        return n + sum(t.numel() * 4 for t in self.state.values())
