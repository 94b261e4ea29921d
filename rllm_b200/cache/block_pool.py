"""The pool of cache pages of one group of layers: reference counts, a free
list, and the table from a content hash to the page that holds it.

The pool itself is C++ (``native/csrc/cache_core.cc``); this class is its
Python face.  Semantics follow the reference's ``BlockPool``
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

import ctypes
from ctypes import c_char_p, c_int, c_void_p
from typing import List, Optional

from ..native import load_library


class PagePoolError(RuntimeError):
    pass


RC_NOT_HELD, RC_BUSY, RC_UNKNOWN_REQ, RC_DUPLICATE_REQ, RC_BADARG, RC_CHECK_FAILED = -2, -3, -4, -5, -6, -7
_lib = None


def core():
    """The C++ library with its argument and result types set."""
    global _lib
    if _lib is None:
        lib = load_library("cache_core")
        for name in ("rllm_pool_new", "rllm_cache_new", "rllm_cache_pool"):
            getattr(lib, name).restype = c_void_p
        for name in ("rllm_page_hashes", "rllm_cache_match_prefix", "rllm_cache_adopt_prefix", "rllm_cache_max_tokens"):
            getattr(lib, name).restype = ctypes.c_longlong
        lib.rllm_pool_delete.restype = None
        lib.rllm_cache_delete.restype = None
        _lib = lib
    return _lib


def _hash16(content_hash: bytes) -> bytes:
    if len(content_hash) > 16:
        raise ValueError("a content hash has at most 16 bytes")
    return content_hash.ljust(16, b"\0")


class _Refcounts:
    """``pool.refcount[page]``"""

    def __init__(self, pool: "BlockPool"):
        self._pool = pool

    def __getitem__(self, page: int) -> int:
        n = core().rllm_pool_refcount(self._pool._h, c_int(page))
        if n < 0:
            raise IndexError(page)
        return n

    def __len__(self) -> int:
        return self._pool.num_pages

    def __iter__(self):
        return (self[p] for p in range(len(self)))


class BlockPool:
    def __init__(self, num_pages: int, _handle=None):
        if _handle is None:
            if num_pages < 1:
                raise ValueError("a pool needs at least one page")
            self._h = c_void_p(core().rllm_pool_new(c_int(num_pages)))
            self._owned = True
        else:
            self._h = c_void_p(_handle)        # a pool inside a cache manager, which owns it
            self._owned = False
        self.num_pages = int(core().rllm_pool_num_pages(self._h))
        self.refcount = _Refcounts(self)

    def __del__(self):
        if getattr(self, "_owned", False) and _lib is not None:
            _lib.rllm_pool_delete(self._h)
            self._owned = False

    # -- counts -----------------------------------------------------------
    @property
    def num_free(self) -> int:
        return int(core().rllm_pool_num_free(self._h))

    @property
    def num_active(self) -> int:
        return self.num_pages - self.num_free

    @property
    def num_cached(self) -> int:
        return int(core().rllm_pool_num_cached(self._h))

    # -- allocation -------------------------------------------------------
    def allocate(self) -> Optional[int]:
        page = core().rllm_pool_allocate(self._h)
        return None if page < 0 else int(page)

    def incref(self, page: int) -> None:
        if core().rllm_pool_incref(self._h, c_int(page)) < 0:
            raise PagePoolError(f"page {page} is not held")

    def free(self, page: int) -> None:
        if core().rllm_pool_free(self._h, c_int(page)) < 0:
            raise PagePoolError(f"page {page} is freed but not held")

    def is_shared(self, page: int) -> bool:
        return self.refcount[page] > 1

    def copy_on_write(self, page: int) -> Optional[int]:
        """The page to write to in place of ``page``: ``page`` itself if it has one owner;
        else this owner's reference is dropped and a fresh page is returned, into which
        the caller copies the data (block_pool.rs:292-302).  None: no page is free."""
        got = core().rllm_pool_copy_on_write(self._h, c_int(page))
        if got == RC_NOT_HELD:
            raise PagePoolError(f"page {page} is not held")
        return None if got < 0 else int(got)

    # -- content hashes ---------------------------------------------------
    def register(self, page: int, content_hash: bytes) -> None:
        """Make a held, completely written page findable by its content."""
        if core().rllm_pool_register(self._h, c_int(page), c_char_p(_hash16(content_hash))) < 0:
            raise PagePoolError(f"page {page} is not held")

    def peek(self, content_hash: bytes) -> Optional[int]:
        """The page with this content, without taking a reference."""
        page = core().rllm_pool_peek(self._h, c_char_p(_hash16(content_hash)))
        return None if page < 0 else int(page)

    def acquire_cached(self, content_hash: bytes) -> Optional[int]:
        """Take a reference to the page with this content, reviving it from the
        free list if need be (block_pool.rs:329-348)."""
        page = core().rllm_pool_acquire_cached(self._h, c_char_p(_hash16(content_hash)))
        return None if page < 0 else int(page)

    def reset_prefix_cache(self) -> None:
        """Forget all content hashes; refused while hashed pages are held
        (block_pool.rs:367-385)."""
        if core().rllm_pool_reset_prefix_cache(self._h) < 0:
            raise PagePoolError("cannot reset the prefix cache while hashed pages are held")

    # -- invariants, for tests -----------------------------------------------
    def check(self) -> None:
        why = ctypes.create_string_buffer(256)
        if core().rllm_pool_check(self._h, why, c_int(256)) < 0:
            raise AssertionError(why.value.decode())
