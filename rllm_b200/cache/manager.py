"""The cache manager: pages of keys and values with a block table for each
request, per group of layers, and slots for per-request state of fixed size.

A model's mixers declare what they keep (``KVPagesNeed``: all keys, or a
window of them; ``StateNeed``: a fixed-size state).  Runs with the same need
form a group.  Every paged group has a pool of pages of its own and every
request a block table per paged group; every request also holds one state
slot, whose index addresses the storage of all state groups (a model without
stateful mixers still gets slots: the engine keeps per-request sampling state
there).  Pages and the slot are given back when a request ends or is
preempted; pages of a windowed group are given back as soon as the window has
passed them; what is given back is used again.

Like the reference's ``KVCacheManager`` (crates/rllm-cache/src/manager.rs:34-269)
allocation is all-or-nothing (:132-166), block tables only grow (:162-163),
and full pages can be shared between requests with the same prefix through
chained content hashes (crates/rllm-cache/src/prefix.rs:43-71; lookup
manager.rs:80-121, registration after the compute :184-210).  Unlike it, a
prefix lookup takes no references until the request is admitted, pages are
hashed only after their keys exist, and a prompt that is cached completely
still computes its last page so that there is a logit to sample from
(the intent of prefix.rs:73-86).  Prefix sharing needs a model whose only
cache group keeps all keys; with windows or state it is switched off.

This is host-side bookkeeping only; the storage lives in ``CacheStorage``.
"""
from __future__ import annotations

import hashlib
import struct
from typing import Dict, Hashable, List, Optional, Sequence

from ..parts.spec import KVPagesNeed, StateNeed
from .block_pool import BlockPool, PagePoolError


class NoCapacity(RuntimeError):
    """No state slot is free."""


def page_hashes(tokens: Sequence[int], page_size: int, salt: bytes = b"",
                start: int = 0, parent: bytes = b"") -> List[bytes]:
    """Chained hashes of the full pages of ``tokens`` from page ``start`` on:
    h_k = H(h_{k-1} | tokens of page k | salt), the first parent empty
    (crates/rllm-cache/src/prefix.rs:43-71)."""
    out = []
    for k in range(start, len(tokens) // page_size):
        chunk = tokens[k * page_size:(k + 1) * page_size]
        h = hashlib.sha256()
        h.update(parent)
        h.update(struct.pack(f"<{page_size}q", *chunk))
        h.update(salt)
        parent = h.digest()[:16]
        out.append(parent)
    return out


class _Request:
    __slots__ = ("slot", "tables", "released", "hashes", "registered")

    def __init__(self, slot: int, num_groups: int):
        self.slot = slot
        self.tables: List[List[int]] = [[] for _ in range(num_groups)]
        self.released: List[int] = [0] * num_groups   # leading pages given back (windows)
        self.hashes: List[bytes] = []                 # content hashes of this request's full pages
        self.registered = 0                           # pages already made findable


class CacheManager:
    def __init__(self, needs: Sequence[object], page_size: int, num_pages, max_seqs: int,
                 enable_prefix_caching: bool = False):
        if page_size < 1 or max_seqs < 1:
            raise ValueError("page_size and max_seqs must be >= 1")
        self.needs = list(needs)
        self.page_size = page_size
        self.max_seqs = max_seqs
        self.paged = [g for g, n in enumerate(self.needs) if isinstance(n, KVPagesNeed)]
        self.stateful = [g for g, n in enumerate(self.needs) if isinstance(n, StateNeed)]
        counts = list(num_pages) if isinstance(num_pages, (list, tuple)) else [num_pages] * len(self.paged)
        if len(counts) != len(self.paged):
            raise ValueError("num_pages: one count per paged group")
        self.pools: Dict[int, BlockPool] = {g: BlockPool(c) for g, c in zip(self.paged, counts)}
        self.requests: Dict[Hashable, _Request] = {}
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self.fresh_slots: List[int] = []   # slots handed out since the last take_fresh_slots()
        only_full = (len(self.paged) == 1 and not self.stateful
                     and self.needs[self.paged[0]].window is None)
        self.prefix_caching = bool(enable_prefix_caching and only_full)

    # -- admission and release -------------------------------------------------
    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def admit(self, req: Hashable) -> int:
        if req in self.requests:
            raise KeyError(f"request {req!r} is already admitted")
        if not self._free_slots:
            raise NoCapacity("no free state slot")
        slot = self._free_slots.pop()
        self.requests[req] = _Request(slot, len(self.needs))
        self.fresh_slots.append(slot)
        return slot

    def take_fresh_slots(self) -> List[int]:
        """Slots handed out since the last call: their state must be zeroed
        before the next step."""
        out, self.fresh_slots = self.fresh_slots, []
        return out

    def free(self, req: Hashable) -> None:
        r = self.requests.pop(req, None)
        if r is None:
            return
        for g in self.paged:
            for page in r.tables[g]:
                if page >= 0:
                    self.pools[g].free(page)
        self._free_slots.append(r.slot)
        if r.slot in self.fresh_slots:
            self.fresh_slots.remove(r.slot)

    def slot(self, req: Hashable) -> int:
        return self.requests[req].slot

    def table(self, req: Hashable, group: int) -> List[int]:
        return self.requests[req].tables[group]

    # -- pages ------------------------------------------------------------------
    def _first_needed_page(self, group: int, first_query_pos: int) -> int:
        window = self.needs[group].window
        if window is None:
            return 0
        return max(0, first_query_pos - window + 1) // self.page_size

    def release_behind_window(self, req: Hashable, first_query_pos: int) -> int:
        """Give back the pages that no query at or after ``first_query_pos`` can
        see.  Returns how many pages were given back."""
        r = self.requests[req]
        n = 0
        for g in self.paged:
            upto = min(self._first_needed_page(g, first_query_pos), len(r.tables[g]))
            for k in range(r.released[g], upto):
                if r.tables[g][k] >= 0:
                    self.pools[g].free(r.tables[g][k])
                    r.tables[g][k] = -1
                    n += 1
            r.released[g] = max(r.released[g], upto)
        return n

    def pages_needed(self, req: Hashable, first_query_pos: int, num_tokens: int) -> Dict[int, int]:
        """New pages per paged group that ``ensure`` would take."""
        r = self.requests[req]
        want = -(-num_tokens // self.page_size)
        out = {}
        for g in self.paged:
            have = len(r.tables[g])
            first = max(self._first_needed_page(g, first_query_pos), have)
            out[g] = max(0, want - first)
        return out

    def ensure(self, req: Hashable, first_query_pos: int, num_tokens: int) -> bool:
        """Make sure the request has pages for positions < ``num_tokens`` that
        queries from ``first_query_pos`` on can see, in every paged group.
        All or nothing: on False no page was taken
        (crates/rllm-cache/src/manager.rs:132-166)."""
        self.release_behind_window(req, first_query_pos)
        need = self.pages_needed(req, first_query_pos, num_tokens)
        if any(self.pools[g].num_free < n for g, n in need.items()):
            return False
        r = self.requests[req]
        want = -(-num_tokens // self.page_size)
        for g in self.paged:
            first = self._first_needed_page(g, first_query_pos)
            while len(r.tables[g]) < want:
                k = len(r.tables[g])
                if k < first:           # behind the window from the start: never held
                    r.tables[g].append(-1)
                    r.released[g] = k + 1
                else:
                    page = self.pools[g].allocate()
                    assert page is not None
                    r.tables[g].append(page)
        return True

    def fits_at_all(self, num_tokens: int) -> bool:
        """Could one request of ``num_tokens`` tokens ever be held?"""
        want = -(-num_tokens // self.page_size)
        for g in self.paged:
            window = self.needs[g].window
            if window is not None:
                want_g = min(want, -(-(window + self.page_size) // self.page_size) + 1)
            else:
                want_g = want
            if want_g > self.pools[g].num_pages:
                return False
        return True

    # -- prefix sharing ------------------------------------------------------------
    def match_prefix(self, tokens: Sequence[int]) -> int:
        """How many leading tokens of ``tokens`` lie in findable pages.  Takes no
        reference.  A prompt that is cached completely reports one page less."""
        if not self.prefix_caching:
            return 0
        pool = self.pools[self.paged[0]]
        n = 0
        for h in page_hashes(tokens, self.page_size):
            if pool.peek(h) is None:
                break
            n += 1
        if n and n * self.page_size >= len(tokens):
            n -= 1
        return n * self.page_size

    def adopt_prefix(self, req: Hashable, tokens: Sequence[int]) -> int:
        """Give a newly admitted request the findable pages of its prefix.
        Returns the number of tokens it need not compute."""
        if not self.prefix_caching:
            return 0
        r = self.requests[req]
        g = self.paged[0]
        if r.tables[g]:
            raise PagePoolError("adopt_prefix on a request that already holds pages")
        pool = self.pools[g]
        limit = (len(tokens) - 1) // self.page_size        # keep at least one token to compute
        hashes = page_hashes(tokens, self.page_size)[:limit]
        for h in hashes:
            page = pool.acquire_cached(h)
            if page is None:
                break
            r.tables[g].append(page)
        n = len(r.tables[g])
        r.hashes = hashes[:n]
        r.registered = n
        return n * self.page_size

    def register_computed(self, req: Hashable, tokens: Sequence[int], num_computed: int) -> None:
        """Make the pages findable whose keys now exist for all their tokens
        (crates/rllm-cache/src/manager.rs:184-210)."""
        if not self.prefix_caching:
            return
        r = self.requests[req]
        g = self.paged[0]
        full = min(num_computed, len(tokens)) // self.page_size
        if full > len(r.hashes):
            parent = r.hashes[-1] if r.hashes else b""
            r.hashes += page_hashes(tokens[:full * self.page_size], self.page_size,
                                    start=len(r.hashes), parent=parent)
        pool = self.pools[g]
        for k in range(r.registered, full):
            pool.register(r.tables[g][k], r.hashes[k])
        r.registered = max(r.registered, full)

    # -- statistics and invariants -----------------------------------------------------
    def usage(self) -> dict:
        return {
            "num_requests": len(self.requests),
            "free_slots": len(self._free_slots),
            "groups": {g: {"total": p.num_pages, "free": p.num_free, "active": p.num_active,
                           "cached": p.num_cached} for g, p in self.pools.items()},
        }

    def num_free_pages(self, group: Optional[int] = None) -> int:
        if group is None:
            return min((p.num_free for p in self.pools.values()), default=0)
        return self.pools[group].num_free

    def check(self) -> None:
        """No page lost, held twice without a matching count, or freed twice."""
        for g in self.paged:
            pool = self.pools[g]
            pool.check()
            held: Dict[int, int] = {}
            for r in self.requests.values():
                for page in r.tables[g]:
                    if page >= 0:
                        held[page] = held.get(page, 0) + 1
            for page in range(pool.num_pages):
                assert pool.refcount[page] == held.get(page, 0), \
                    f"group {g} page {page}: count {pool.refcount[page]}, held by {held.get(page, 0)}"
        slots = [r.slot for r in self.requests.values()] + self._free_slots
        assert sorted(slots) == list(range(self.max_seqs)), "a state slot is lost or held twice"
