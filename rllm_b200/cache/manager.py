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
(the intent of prefix.rs:73-86).  With several paged groups every group keeps
the hashes of its own pages, and a request takes over the longest prefix for
which every group still has what the request's next query can see: all pages
where every key is kept, those that reach into the window where a window is
kept (the pages before them are left out of its table, as if the window had
passed them).  State of fixed size cannot be taken over from pages: with a
group of that kind prefix sharing is switched off.

This is host-side bookkeeping only; the storage lives in ``CacheStorage``.  The
bookkeeping itself is C++ (``native/csrc/cache_core.cc``); this class is its
Python face: it maps request ids (any hashable) to the integers the C++ side
knows and turns its return codes into exceptions.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_longlong, c_void_p
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from ..parts.spec import KVPagesNeed, StateNeed
from .block_pool import RC_DUPLICATE_REQ, RC_NOT_HELD, RC_UNKNOWN_REQ, BlockPool, PagePoolError, core


class NoCapacity(RuntimeError):
    """No state slot is free."""


def _tokens(tokens: Sequence[int]) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(tokens, dtype=np.int64))


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(c_void_p)


def page_hashes(tokens: Sequence[int], page_size: int, salt: bytes = b"",
                start: int = 0, parent: bytes = b"") -> List[bytes]:
    """Chained hashes of the full pages of ``tokens`` from page ``start`` on:
    h_k = SHA-256(h_{k-1} | tokens of page k as little-endian int64 | salt) cut to 16
    bytes, the first parent empty (crates/rllm-cache/src/prefix.rs:43-71)."""
    t = _tokens(tokens)
    n = max(0, len(t) // page_size - start)
    out = ctypes.create_string_buffer(16 * max(n, 1))
    got = core().rllm_page_hashes(_ptr(t), c_longlong(len(t)), c_int(page_size), c_char_p(salt), c_int(len(salt)),
                                  c_int(start), c_char_p(parent) if parent else None, out, c_longlong(n))
    if got < 0:
        raise ValueError("page_hashes: bad arguments")
    return [out.raw[16 * i:16 * i + 16] for i in range(got)]


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
        G = len(self.needs)
        kinds = (c_int * max(G, 1))(*[0 if g in self.paged else 1 for g in range(G)])
        windows = (c_int * max(G, 1))(*[(-1 if getattr(n, "window", None) is None else int(n.window))
                                        for n in self.needs])
        per_group = [0] * G
        for g, c in zip(self.paged, counts):
            if c < 1:
                raise ValueError("a pool needs at least one page")
            per_group[g] = int(c)
        h = core().rllm_cache_new(c_int(G), kinds, windows, (c_int * max(G, 1))(*per_group), c_int(page_size),
                                  c_int(max_seqs), c_int(1 if enable_prefix_caching else 0))
        if not h:
            raise ValueError("CacheManager: bad sizes")
        self._h = c_void_p(h)
        self.pools: Dict[int, BlockPool] = {
            g: BlockPool(0, _handle=core().rllm_cache_pool(self._h, c_int(g))) for g in self.paged}
        self.requests: Dict[Hashable, int] = {}       # request id -> the integer the C++ side knows it by
        self._next_id = 0
        self.prefix_caching = bool(core().rllm_cache_prefix_caching(self._h))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h is not None:
            try:
                core().rllm_cache_delete(h)
            except Exception:
                pass
            self._h = None

    def _id(self, req: Hashable) -> c_longlong:
        return c_longlong(self.requests[req])

    # -- admission and release -------------------------------------------------
    def has_free_slot(self) -> bool:
        return core().rllm_cache_num_free_slots(self._h) > 0

    def admit(self, req: Hashable) -> int:
        if req in self.requests:
            raise KeyError(f"request {req!r} is already admitted")
        rid = self._next_id
        slot = core().rllm_cache_admit(self._h, c_longlong(rid))
        if slot == RC_DUPLICATE_REQ:
            raise KeyError(f"request {req!r} is already admitted")
        if slot < 0:
            raise NoCapacity("no free state slot")
        self._next_id += 1
        self.requests[req] = rid
        return int(slot)

    @property
    def fresh_slots(self) -> int:
        """How many slots were handed out since the last ``take_fresh_slots``."""
        return int(core().rllm_cache_num_fresh_slots(self._h))

    def take_fresh_slots(self) -> List[int]:
        """Slots handed out since the last call: their state must be zeroed
        before the next step."""
        n = self.fresh_slots
        if not n:
            return []
        buf = (c_int * n)()
        got = core().rllm_cache_take_fresh_slots(self._h, buf, c_int(n))
        return [int(buf[i]) for i in range(got)]

    def free(self, req: Hashable) -> None:
        rid = self.requests.pop(req, None)
        if rid is not None:
            core().rllm_cache_free(self._h, c_longlong(rid))

    def fork(self, parent: Hashable, child: Hashable, num_tokens: int):
        """Admit ``child`` as a copy of the first ``num_tokens`` tokens of ``parent``
        (crates/rllm-cache/src/manager.rs:220-245): it shares the parent's full pages by
        reference count and gets a page of its own for the partly filled last one, and a
        state slot of its own.  Returns (copies, (parent slot, child slot)) with copies =
        [(group, parent's page, child's page)]: the caller copies those pages and the
        state slot on the device (``CacheStorage.copy_for_fork``) before either request
        runs again.  None if a slot or a page is missing; nothing was taken then."""
        if child in self.requests:
            raise KeyError(f"request {child!r} is already admitted")
        cap = 3 * max(1, len(self.paged))
        buf = (c_int * cap)()
        n = c_int(0)
        rid = self._next_id
        slot = core().rllm_cache_fork(self._h, self._id(parent), c_longlong(rid), c_longlong(num_tokens), buf,
                                      c_int(cap), ctypes.byref(n))
        if slot == -1:
            return None
        if slot == RC_NOT_HELD:
            raise PagePoolError(f"fork: request {parent!r} does not hold pages for {num_tokens} tokens")
        if slot < 0:
            raise ValueError(f"fork: bad arguments ({slot})")
        self._next_id += 1
        self.requests[child] = rid
        copies = [(int(buf[3 * i]), int(buf[3 * i + 1]), int(buf[3 * i + 2])) for i in range(n.value)]
        return copies, (self.slot(parent), int(slot))

    def slot(self, req: Hashable) -> int:
        return int(core().rllm_cache_slot(self._h, self._id(req)))

    def table_len(self, req: Hashable, group: int) -> int:
        return int(core().rllm_cache_table_len(self._h, self._id(req), c_int(group)))

    def table(self, req: Hashable, group: int) -> List[int]:
        """A copy of the request's block table in this group (-1: a page given back)."""
        n = self.table_len(req, group)
        if n <= 0:
            return []
        buf = (c_int * n)()
        core().rllm_cache_table(self._h, self._id(req), c_int(group), buf, c_int(n))
        return list(buf)

    def pack_tables(self, reqs: Sequence[Hashable], group: int, out: np.ndarray) -> None:
        """Row i of ``out`` (int32 [len(reqs), width], C-contiguous) = the table of reqs[i], -1 behind its end."""
        assert out.dtype == np.int32 and out.flags.c_contiguous and out.shape[0] >= len(reqs)
        ids = np.fromiter((self.requests[r] for r in reqs), dtype=np.int64, count=len(reqs))
        rc = core().rllm_cache_pack_tables(self._h, _ptr(ids), c_int(len(reqs)), c_int(group), _ptr(out),
                                           c_int(out.shape[1]))
        if rc < 0:
            raise KeyError("pack_tables: a request is not admitted")

    # -- pages ------------------------------------------------------------------
    def release_behind_window(self, req: Hashable, first_query_pos: int) -> int:
        """Give back the pages that no query at or after ``first_query_pos`` can
        see.  Returns how many pages were given back."""
        return int(core().rllm_cache_release_behind_window(self._h, self._id(req), c_longlong(first_query_pos)))

    def pages_needed(self, req: Hashable, first_query_pos: int, num_tokens: int) -> Dict[int, int]:
        """New pages per paged group that ``ensure`` would take."""
        rid = self._id(req)
        return {g: int(core().rllm_cache_pages_needed(self._h, rid, c_int(g), c_longlong(first_query_pos),
                                                      c_longlong(num_tokens))) for g in self.paged}

    def ensure(self, req: Hashable, first_query_pos: int, num_tokens: int) -> bool:
        """Make sure the request has pages for positions < ``num_tokens`` that
        queries from ``first_query_pos`` on can see, in every paged group.
        All or nothing: on False no page was taken
        (crates/rllm-cache/src/manager.rs:132-166)."""
        rc = core().rllm_cache_ensure(self._h, self._id(req), c_longlong(first_query_pos), c_longlong(num_tokens))
        if rc < 0:
            raise KeyError(req)
        return bool(rc)

    def max_tokens(self, req: Hashable, first_query_pos: int) -> int:
        """The largest ``num_tokens`` for which ``ensure(req, first_query_pos, num_tokens)``
        would succeed now.  Gives back the pages behind the window first, as ``ensure`` does."""
        n = core().rllm_cache_max_tokens(self._h, self._id(req), c_longlong(first_query_pos))
        if n < 0:
            raise KeyError(req)
        return int(n)

    def fits_at_all(self, num_tokens: int) -> bool:
        """Could one request of ``num_tokens`` tokens ever be held?"""
        return bool(core().rllm_cache_fits_at_all(self._h, c_longlong(num_tokens)))

    # -- prefix sharing ------------------------------------------------------------
    def match_prefix(self, tokens: Sequence[int]) -> int:
        """How many leading tokens of ``tokens`` lie in findable pages.  Takes no
        reference.  A prompt that is cached completely reports one page less."""
        if not self.prefix_caching:
            return 0
        t = _tokens(tokens)
        return int(core().rllm_cache_match_prefix(self._h, _ptr(t), c_longlong(len(t))))

    def adopt_prefix(self, req: Hashable, tokens: Sequence[int]) -> int:
        """Give a newly admitted request the findable pages of its prefix.
        Returns the number of tokens it need not compute."""
        if not self.prefix_caching:
            return 0
        t = _tokens(tokens)
        n = core().rllm_cache_adopt_prefix(self._h, self._id(req), _ptr(t), c_longlong(len(t)))
        if n == RC_NOT_HELD:
            raise PagePoolError("adopt_prefix on a request that already holds pages")
        if n == RC_UNKNOWN_REQ:
            raise KeyError(req)
        return int(n)

    def register_computed(self, req: Hashable, tokens: Sequence[int], num_computed: int) -> None:
        """Make the pages findable whose keys now exist for all their tokens
        (crates/rllm-cache/src/manager.rs:184-210)."""
        if not self.prefix_caching:
            return
        t = _tokens(tokens)
        core().rllm_cache_register_computed(self._h, self._id(req), _ptr(t), c_longlong(len(t)),
                                            c_longlong(num_computed))

    def reset_prefix_cache(self) -> None:
        """Forget the hashes of all pages (crates/rllm-cache/src/block_pool.rs:367-385); refused while
        a request holds a hashed page."""
        if any(p.num_active for p in self.pools.values()):
            raise PagePoolError("reset_prefix_cache while requests hold pages")
        for p in self.pools.values():
            p.reset_prefix_cache()

    # -- statistics and invariants -----------------------------------------------------
    def usage(self) -> dict:
        return {
            "num_requests": len(self.requests),
            "free_slots": int(core().rllm_cache_num_free_slots(self._h)),
            "groups": {g: {"total": p.num_pages, "free": p.num_free, "active": p.num_active,
                           "cached": p.num_cached} for g, p in self.pools.items()},
        }

    def num_free_pages(self, group: Optional[int] = None) -> int:
        if group is None:
            return min((p.num_free for p in self.pools.values()), default=0)
        return self.pools[group].num_free

    def check(self) -> None:
        """No page lost, held twice without a matching count, or freed twice."""
        why = ctypes.create_string_buffer(256)
        if core().rllm_cache_check(self._h, why, c_int(256)) < 0:
            raise AssertionError(why.value.decode())
        assert core().rllm_cache_num_requests(self._h) == len(self.requests)
