"""The pool of cache pages of one group of layers: reference counts, a free
list, and the table from a content hash to the page that holds it.

Semantics follow the reference's ``BlockPool``
(crates/rllm-cache/src/block_pool.rs:128-406): a page is handed out with
reference count 1; ``free`` decrements and at 0 the page joins the free list
*keeping its hash*, so a later request with the same prefix can revive it
(:247-261, :307-348); ``allocate`` prefers free pages without a hash and only
then evicts the least recently freed hashed page, dropping its hash
(:198-241).  Freeing a page that is not held is an error here (the reference
ignores it).  There is no reserved null page: "no page" is -1 in a block
table.
"""
from __future__ import annotations

from collections import OrderedDict, deque
from typing import Deque, Dict, List, Optional


class PagePoolError(RuntimeError):
    pass


class BlockPool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self.refcount: List[int] = [0] * num_pages
        self.hash_of: List[Optional[bytes]] = [None] * num_pages
        self.page_of: Dict[bytes, int] = {}
        # free pages without a hash: last in, first out
        self._free_plain: Deque[int] = deque(range(num_pages - 1, -1, -1))
        # free pages that still hold findable content, least recently freed first
        self._free_cached: "OrderedDict[int, None]" = OrderedDict()

    # -- counts -----------------------------------------------------------
    @property
    def num_free(self) -> int:
        return len(self._free_plain) + len(self._free_cached)

    @property
    def num_active(self) -> int:
        return self.num_pages - self.num_free

    @property
    def num_cached(self) -> int:
        return len(self.page_of)

    # -- allocation -------------------------------------------------------
    def allocate(self) -> Optional[int]:
        if self._free_plain:
            page = self._free_plain.pop()
        elif self._free_cached:
            page, _ = self._free_cached.popitem(last=False)
            self._drop_hash(page)
        else:
            return None
        self.refcount[page] = 1
        return page

    def incref(self, page: int) -> None:
        if self.refcount[page] < 1:
            raise PagePoolError(f"page {page} is not held")
        self.refcount[page] += 1

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages or self.refcount[page] < 1:
            raise PagePoolError(f"page {page} is freed but not held")
        self.refcount[page] -= 1
        if self.refcount[page] == 0:
            if self.hash_of[page] is not None:
                self._free_cached[page] = None
            else:
                self._free_plain.append(page)

    def is_shared(self, page: int) -> bool:
        return self.refcount[page] > 1

    # -- content hashes ---------------------------------------------------
    def register(self, page: int, content_hash: bytes) -> None:
        """Make a held, completely written page findable by its content."""
        if self.refcount[page] < 1:
            raise PagePoolError(f"page {page} is not held")
        if self.hash_of[page] is not None or content_hash in self.page_of:
            return  # already findable (or the same content lives in another page)
        self.hash_of[page] = content_hash
        self.page_of[content_hash] = page

    def peek(self, content_hash: bytes) -> Optional[int]:
        """The page with this content, without taking a reference."""
        return self.page_of.get(content_hash)

    def acquire_cached(self, content_hash: bytes) -> Optional[int]:
        """Take a reference to the page with this content, reviving it from the
        free list if need be (block_pool.rs:329-348)."""
        page = self.page_of.get(content_hash)
        if page is None:
            return None
        if self.refcount[page] == 0:
            del self._free_cached[page]
        self.refcount[page] += 1
        return page

    def reset_prefix_cache(self) -> None:
        """Forget all content hashes; refused while hashed pages are held
        (block_pool.rs:367-385)."""
        if any(self.refcount[p] > 0 for p in self.page_of.values()):
            raise PagePoolError("cannot reset the prefix cache while hashed pages are held")
        for page in list(self._free_cached):
            self._free_plain.append(page)
        self._free_cached.clear()
        for page in self.page_of.values():
            self.hash_of[page] = None
        self.page_of.clear()

    def _drop_hash(self, page: int) -> None:
        h = self.hash_of[page]
        if h is not None:
            del self.page_of[h]
            self.hash_of[page] = None

    # -- invariants, for tests -----------------------------------------------
    def check(self) -> None:
        free = list(self._free_plain) + list(self._free_cached)
        assert len(free) == len(set(free)), "a page is on the free list twice"
        for p in range(self.num_pages):
            assert (self.refcount[p] == 0) == (p in set(free)), f"page {p}: count and free list disagree"
        for h, p in self.page_of.items():
            assert self.hash_of[p] == h
        for p in self._free_plain:
            assert self.hash_of[p] is None
        for p in self._free_cached:
            assert self.hash_of[p] is not None
