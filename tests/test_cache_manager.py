"""The cache manager on the host: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; prefix sharing
(mirrors crates/rllm-cache/src/block_pool.rs:421-635, manager.rs:271-516)."""
import random

import pytest

from rllm_b200.cache import BlockPool, CacheManager, NoCapacity, PagePoolError, page_hashes
from rllm_b200.parts.spec import KVPagesNeed, StateNeed

FULL = KVPagesNeed(2, 16, None)


def test_pool_counts_and_double_free():
    pool = BlockPool(4)
    pages = [pool.allocate() for _ in range(4)]
    assert sorted(pages) == [0, 1, 2, 3] and pool.allocate() is None and pool.num_free == 0
    pool.free(pages[0])
    with pytest.raises(PagePoolError):
        pool.free(pages[0])
    assert pool.num_free == 1 and pool.allocate() == pages[0]
    pool.check()


def test_pool_prefers_pages_without_content_and_evicts_oldest():
    pool = BlockPool(3)
    a, b, c = (pool.allocate() for _ in range(3))
    pool.register(a, b"A"); pool.register(b, b"B")
    pool.free(a); pool.free(b); pool.free(c)
    assert pool.allocate() == c                       # no content: first choice
    assert pool.peek(b"A") == a and pool.peek(b"B") == b
    assert pool.allocate() == a and pool.peek(b"A") is None   # least recently freed content goes first
    assert pool.acquire_cached(b"B") == b and pool.refcount[b] == 1
    pool.check()


def test_shared_page_needs_both_frees():
    pool = BlockPool(2)
    a = pool.allocate()
    pool.register(a, b"A")
    assert pool.acquire_cached(b"A") == a and pool.is_shared(a)
    pool.free(a)
    assert pool.num_free == 1
    pool.free(a)
    assert pool.num_free == 2
    with pytest.raises(PagePoolError):
        pool.free(99)
    assert pool.acquire_cached(b"A") == a
    with pytest.raises(PagePoolError):
        pool.reset_prefix_cache()                     # refused while a hashed page is held
    pool.free(a)
    pool.reset_prefix_cache()
    assert pool.peek(b"A") is None
    pool.check()


def test_all_or_nothing():
    m = CacheManager([FULL], 16, 4, 8)
    m.admit("a"); m.admit("b")
    assert m.ensure("a", 0, 40)                       # 3 pages
    assert not m.ensure("b", 0, 40)                   # needs 3, 1 free: nothing taken
    assert m.num_free_pages() == 1 and m.table("b", 0) == []
    assert m.ensure("b", 0, 16)
    m.free("a")
    assert m.ensure("b", 16, 60)
    m.check()


def test_slots():
    m = CacheManager([FULL], 16, 4, 2)
    s0, s1 = m.admit("a"), m.admit("b")
    assert {s0, s1} == {0, 1} and sorted(m.take_fresh_slots()) == [0, 1]
    with pytest.raises(NoCapacity):
        m.admit("c")
    m.free("a")
    assert m.admit("c") == s0 and m.take_fresh_slots() == [s0]
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    needs = [FULL, KVPagesNeed(1, 32, 24), StateNeed((4,))]
    m = CacheManager(needs, 8, [40, 12], 5)
    live = {}
    for step in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{step}"
            m.admit(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = live[rid] + rng.choice([1, 1, 1, 2, 7, 23])
            if m.ensure(rid, live[rid], n):
                live[rid] = n
                tb = m.table(rid, 1)          # the windowed group holds only what queries can still see
                held = [k for k, p in enumerate(tb) if p >= 0]
                assert all(k * 8 + 7 >= max(0, live[rid] - 1 - 24 + 1) - 23 for k in held)
        elif op < 0.88 and live and len(live) < 5:
            src, dst = rng.choice(list(live)), f"f{step}"
            upto = rng.randint(0, live[src])
            try:
                if m.fork(src, dst, upto) is not None:
                    live[dst] = upto
            except PagePoolError:
                assert upto < live[src]       # refused: the window has passed pages the child would need
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check()
    for rid in list(live):
        m.free(rid)
    m.check()
    assert m.num_free_pages(0) == 40 and m.num_free_pages(1) == 12 and m.usage()["free_slots"] == 5


def test_window_gives_pages_back_and_reuses_them():
    m = CacheManager([KVPagesNeed(1, 16, 10)], 4, 5, 2)
    m.admit("a")
    pos, seen = 0, set()
    while pos < 200:
        assert m.ensure("a", pos, pos + 3), pos         # 5 pages are enough for ever
        pos += 3
        tb = m.table("a", 0)
        seen.update(p for p in tb if p >= 0)
        first_needed = max(0, pos - 3 - 10 + 1) // 4
        assert all(p == -1 for p in tb[:first_needed]) and all(p >= 0 for p in tb[first_needed:])
    assert seen <= {0, 1, 2, 3, 4} and len(m.table("a", 0)) == 51      # 51 pages went through 5
    m.check()


def test_a_prompt_that_starts_behind_its_window_holds_no_early_pages():
    m = CacheManager([KVPagesNeed(1, 16, 8)], 4, 4, 1)
    m.admit("a")
    assert m.ensure("a", 0, 6)
    assert m.ensure("a", 6, 40) is False               # one portion of 34 tokens sees 8 + 34 keys: 11 pages
    assert m.ensure("a", 6, 14)
    m.check()


def test_page_hashes_are_sha256_chains():
    """The C++ side's own SHA-256 against hashlib: h_k = SHA-256(h_{k-1} | tokens as little-endian int64 | salt)
    cut to 16 bytes, for pages of several sizes (message lengths around the padding's edge cases)."""
    import hashlib
    import struct
    for page in (1, 3, 6, 7, 8, 16, 55):
        toks = [(i * 2654435761) % 100003 - 7 for i in range(page * 5 + 2)]
        for salt in (b"", b"s", b"a longer salt than one block of the hash function, to cross 64 bytes at once"):
            parent = b""
            got = page_hashes(toks, page, salt=salt)
            assert len(got) == len(toks) // page
            for k, h in enumerate(got):
                m = hashlib.sha256()
                m.update(parent)
                m.update(struct.pack(f"<{page}q", *toks[k * page:(k + 1) * page]))
                m.update(salt)
                parent = m.digest()[:16]
                assert h == parent, (page, k)


def test_page_hashes_chain():
    toks = list(range(40))
    h = page_hashes(toks, 16)
    assert len(h) == 2 and h[0] != h[1]
    assert page_hashes(toks[:16] + [99] + toks[17:], 16)[0] == h[0]
    assert page_hashes([1] + toks[1:], 16)[1] != h[1]        # a page's hash covers all pages before it
    assert page_hashes(toks, 16, salt=b"x")[0] != h[0]
    assert page_hashes(toks, 16, start=1, parent=h[0]) == h[1:]


def test_prefix_sharing():
    m = CacheManager([FULL], 4, 16, 4, enable_prefix_caching=True)
    toks = list(range(100, 118))                       # 4 full pages + 2 tokens
    m.admit("a")
    assert m.match_prefix(toks) == 0 and m.adopt_prefix("a", toks) == 0
    assert m.ensure("a", 0, 18)
    m.register_computed("a", toks, 10)                 # only 2 pages have all their keys
    assert m.match_prefix(toks) == 8                   # a lookup takes no reference
    m.check()
    m.register_computed("a", toks, 18)
    m.admit("b")
    assert m.adopt_prefix("b", toks + [7, 8, 9]) == 16
    assert m.table("b", 0) == m.table("a", 0)[:4]
    m.check()
    m.free("a")
    m.check()
    m.admit("c")
    assert m.match_prefix(toks[:16]) == 12             # wholly cached: the last page is computed again
    assert m.adopt_prefix("c", toks[:16]) == 12
    m.free("b"); m.free("c")
    m.check()
    assert m.num_free_pages() == 16
    m.admit("d")
    assert m.adopt_prefix("d", toks) == 16             # freed pages stay findable until they are reused
    m.check()


def test_prefix_sharing_is_off_with_state():
    assert not CacheManager([FULL, StateNeed((2,))], 4, 4, 1, enable_prefix_caching=True).prefix_caching
    assert CacheManager([KVPagesNeed(1, 16, 8)], 4, 4, 1, enable_prefix_caching=True).prefix_caching


def test_prefix_sharing_with_a_window_takes_what_the_next_query_sees():
    """Two groups, one keeps all keys, one a window of 6 (pages of 4).  A request that finds its prefix takes all
    pages of the first group and, of the second, only those that reach into the window of its first query."""
    win = KVPagesNeed(1, 16, 6)
    m = CacheManager([FULL, win], 4, [16, 8], 3, enable_prefix_caching=True)
    toks = list(range(100, 130))                       # 7 full pages + 2 tokens
    m.admit("a")
    pos = 0
    for n in (9, 9, 12):                               # portions; the window gives pages back on the way
        assert m.ensure("a", pos, pos + n)
        pos += n
        m.register_computed("a", toks, pos)
    assert m.table("a", 1)[:3] == [-1, -1, -1]
    m.check()
    # 28 tokens in full pages, the prompt has 30: 7 pages can be taken; the query at 28 sees keys 23..: pages 5, 6
    assert m.match_prefix(toks) == 28
    m.admit("b")
    assert m.adopt_prefix("b", toks) == 28
    assert m.table("b", 0) == m.table("a", 0)[:7]
    assert m.table("b", 1) == [-1] * 5 + m.table("a", 1)[5:7]
    m.check()
    assert m.ensure("b", 28, 30) and m.ensure("b", 30, 31)
    m.free("a")
    m.check()
    # pages that the window gave back stay findable until they are used again: a shorter prompt finds them
    assert m.match_prefix(toks[:14]) == 12             # 3 pages; the query at 12 sees 7..: pages 1, 2
    m.admit("c")
    assert m.adopt_prefix("c", toks[:14]) == 12
    assert m.table("c", 1)[0] == -1 and all(p >= 0 for p in m.table("c", 1)[1:3])
    m.check()
    m.free("b"); m.free("c")
    m.check()
    assert m.num_free_pages(0) == 16 and m.num_free_pages(1) == 8
    # once the window group's pages have been used again, only a shorter prefix (or none) can be taken
    m.admit("d")
    assert m.ensure("d", 0, 30)                        # one portion: every page of the windowed group at once
    assert m.match_prefix(toks) < 28
    k = m.match_prefix(toks) // 4
    m.admit("e")
    assert m.adopt_prefix("e", toks) == 4 * k
    assert all(p >= 0 for p in m.table("e", 0)) and len(m.table("e", 0)) == k
    m.check()
    m.free("d"); m.free("e")
    m.reset_prefix_cache()
    assert m.match_prefix(toks) == 0
    m.check()


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_orders_with_prefix_sharing_over_two_groups(seed):
    """Requests with prompts drawn from a few families run in random portions, end in random order, and take
    over what they find: nothing is lost or held twice, and a request never lacks a page its query sees."""
    rng = random.Random(seed)
    window = 10
    m = CacheManager([FULL, KVPagesNeed(1, 16, window)], 4, [48, 14], 4, enable_prefix_caching=True)
    families = [[rng.randrange(1000) for _ in range(60)] for _ in range(3)]
    live = {}
    hits = 0
    for step in range(800):
        op = rng.random()
        if op < 0.2 and len(live) < 4:
            rid = f"r{step}"
            fam = rng.choice(families)
            toks = fam[:rng.randint(1, 60)] + [rng.randrange(1000) for _ in range(rng.randint(0, 6))]
            expect = m.match_prefix(toks)
            m.admit(rid)
            got = m.adopt_prefix(rid, toks)
            assert got == expect and got % 4 == 0 and got < len(toks)
            hits += got
            live[rid] = [toks, got]
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            toks, pos = live[rid]
            if pos == len(toks):
                toks.append(rng.randrange(1000))       # a generated token
            n = min(len(toks), pos + rng.choice([1, 1, 2, 5, 9]))
            if m.ensure(rid, pos, n):
                for g, w in ((0, None), (1, window)):
                    tb = m.table(rid, g)
                    lo = 0 if w is None else max(0, pos - w + 1) // 4
                    assert all(p >= 0 for p in tb[lo:-(-n // 4)]), (rid, g, pos, n, tb)
                live[rid][1] = n
                m.register_computed(rid, toks, n)
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check()
    for rid in list(live):
        m.free(rid)
    m.check()
    assert hits > 0
    assert m.num_free_pages(0) == 48 and m.num_free_pages(1) == 14


def test_fork_shares_full_pages_and_copies_the_last():
    """crates/rllm-cache/src/manager.rs:220-245 (fork) and block_pool.rs:292-302 (copy on write)."""
    m = CacheManager([FULL, StateNeed((4,))], 8, 6, 3)
    m.admit("a")
    m.take_fresh_slots()
    assert m.ensure("a", 0, 21)                         # pages 0, 1 full, page 2 holds 5 tokens
    pool = m.pools[0]
    copies, slots = m.fork("a", "b", 21)
    ta, tb = m.table("a", 0), m.table("b", 0)
    assert ta[:2] == tb[:2] and ta[2] != tb[2] and copies == [(0, ta[2], tb[2])]
    assert [pool.refcount[p] for p in ta] == [2, 2, 1] and pool.refcount[tb[2]] == 1
    assert slots == (m.slot("a"), m.slot("b")) and slots[0] != slots[1]
    assert m.take_fresh_slots() == []                   # the child's state is a copy, not zeros
    # at a page's edge nothing is copied; beyond what the parent holds is an error
    copies, _ = m.fork("a", "c", 16)
    assert copies == [] and m.table("c", 0) == ta[:2]
    with pytest.raises(Exception, match="does not hold"):
        m.fork("a", "d", 40)
    # no slot left: nothing taken
    free_before = pool.num_free
    assert m.fork("a", "d", 21) is None and pool.num_free == free_before
    m.check()
    # each goes on by itself; the shared pages live until the last owner ends
    assert m.ensure("b", 21, 30) and m.ensure("a", 21, 25)
    m.free("a")
    assert [pool.refcount[p] for p in tb[:2]] == [2, 2]
    m.free("c"); m.free("b")
    m.check()
    assert pool.num_free == 6 and m.usage()["free_slots"] == 3


def test_fork_without_a_free_page_takes_nothing():
    m = CacheManager([FULL], 8, 3, 3)
    m.admit("a")
    assert m.ensure("a", 0, 21)
    assert m.fork("a", "b", 21) is None and "b" not in m.requests and m.usage()["free_slots"] == 2
    assert m.fork("a", "b", 16) is not None             # full pages only: no page needed
    m.check()


def test_fork_behind_a_window_is_refused():
    m = CacheManager([KVPagesNeed(1, 16, 10)], 4, 8, 2)
    m.admit("a")
    assert m.ensure("a", 0, 12) and m.ensure("a", 12, 30) and m.ensure("a", 30, 31)   # keys before 20 are gone
    with pytest.raises(PagePoolError):
        m.fork("a", "b", 8)                                    # a query at 8 would see keys from 0 on
    assert m.fork("a", "b", 31) is not None
    m.check()


def test_pool_copy_on_write():
    pool = BlockPool(2)
    a = pool.allocate()
    assert pool.copy_on_write(a) == a                   # one owner: write in place
    pool.incref(a)
    b = pool.copy_on_write(a)
    assert b is not None and b != a and pool.refcount[a] == 1 and pool.refcount[b] == 1
    pool.incref(a)
    assert pool.copy_on_write(a) is None and pool.refcount[a] == 2      # no page free: nothing changes
    pool.check()


def test_pages_are_given_back_last_page_first():
    """Without hashes the pages of a finished request come back in rising order, so the next request's pages
    follow one another; with hashes the last pages of a finished request are the first to be used again, and
    what stays findable is a prefix."""
    m = CacheManager([FULL], 4, 12, 2)
    m.admit("a")
    assert m.ensure("a", 0, 40)
    first = m.table("a", 0)
    assert first == sorted(first)
    m.free("a")
    m.admit("b")
    assert m.ensure("b", 0, 24)
    assert m.table("b", 0) == first[:6]
    m.free("b")
    m.check()
    c = CacheManager([FULL], 4, 8, 2, enable_prefix_caching=True)
    toks = list(range(200, 232))                       # 8 full pages
    c.admit("a")
    assert c.ensure("a", 0, 32)
    c.register_computed("a", toks, 32)
    pages = c.table("a", 0)
    c.free("a")
    c.admit("b")
    assert c.ensure("b", 0, 12)                         # three pages: taken from the end of a's
    assert sorted(c.table("b", 0)) == sorted(pages[5:])
    assert c.match_prefix(toks) == 20                   # pages 0..4 of the prefix are still findable
    c.free("b")
    c.check()
