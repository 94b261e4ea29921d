"""The scheduler's decisions, on the host, with a scripted step function in
place of the model (the reference's engine tests use a fake executor the same
way: crates/rllm-engine/tests/engine_tests.rs:16-122; scheduler tests:
crates/rllm-scheduler/src/scheduler.rs:650-882)."""
import random

import pytest

from rllm_b200.cache import CacheManager
from rllm_b200.engine.scheduler import (Request, RequestRefused, RequestStatus, Scheduler,
                                        SchedulerConfig)
from rllm_b200.parts.spec import KVPagesNeed
from rllm_b200.sampling import SamplingParams

NEED = KVPagesNeed(2, 16, None)


def make(pages=64, page=16, seqs=8, prefix=False, **cfg):
    cache = CacheManager([NEED], page, pages, seqs, enable_prefix_caching=prefix)
    conf = SchedulerConfig(**{**dict(max_num_seqs=seqs, max_num_batched_tokens=64,
                                     long_prefill_token_threshold=0, max_model_len=4096), **cfg})
    return Scheduler(conf, cache), cache


def req(i, n_prompt, max_tokens=8, first=1000):
    return Request(f"r{i}", list(range(first, first + n_prompt)), SamplingParams(max_tokens=max_tokens),
                   arrival=i, seed=i, max_tokens=max_tokens)


def run_step(s, token=lambda r: 7):
    """What the engine does around schedule(): run, append a token where the
    portion ended at the last known token, finish by length."""
    out = s.schedule()
    s.after_step(out)
    for sc in out.scheduled:
        assert sc.num_tokens >= 1 and sc.start == sc.request.num_computed - sc.num_tokens
        if sc.want_logits:
            sc.request.output_token_ids.append(token(sc.request))
            if len(sc.request.output_token_ids) >= sc.request.max_tokens:
                s.finish(sc.request, RequestStatus.FINISHED_LENGTH)
    s.cache.check()
    return out


def test_fcfs_and_budget():
    s, _ = make(max_num_batched_tokens=50)
    for i, n in enumerate([30, 30, 30]):
        s.add_request(req(i, n))
    out = run_step(s)
    assert [(x.request.request_id, x.start, x.num_tokens, x.want_logits) for x in out.scheduled] == \
        [("r0", 0, 30, True), ("r1", 0, 20, False)]
    out = run_step(s)
    # running first: r0 decodes, r1 finishes its prompt, then r2 gets what is left of the budget
    assert [(x.request.request_id, x.start, x.num_tokens, x.want_logits) for x in out.scheduled] == \
        [("r0", 30, 1, True), ("r1", 20, 10, True), ("r2", 0, 30, True)]
    assert out.num_decode_tokens == 1 and out.num_prefill_tokens == 40


def test_portion_cap_and_logits_only_at_the_end():
    s, _ = make(max_num_batched_tokens=64, long_prefill_token_threshold=16)
    s.add_request(req(0, 40))
    seen = []
    while s.has_work() and len(seen) < 3:
        out = run_step(s)
        seen.append([(x.start, x.num_tokens, x.want_logits) for x in out.scheduled])
    assert seen == [[(0, 16, False)], [(16, 16, False)], [(32, 8, True)]]


def test_a_step_a_few_rows_over_a_row_tile_gives_them_back():
    """Five decoding requests beside a 64-token portion are 69 rows, five over two tiles of 32: the portion
    shrinks to 59.  Nothing is cut where the step is under two tiles, lands on a multiple, is more than a
    quarter tile over, or where the only portion is its prompt's last."""
    s, cache = make(pages=256, max_num_batched_tokens=256, long_prefill_token_threshold=64, step_row_multiple=32)
    for i in range(5):
        s.add_request(req(i, 3, max_tokens=40))
    run_step(s)                                               # five prompts of 3 tokens: 15 rows, under two tiles
    s.add_request(req(9, 300, max_tokens=4))
    out = run_step(s)
    assert [(x.request.request_id, x.start, x.num_tokens, x.want_logits) for x in out.scheduled][-1] == ("r9", 0, 59, False)
    assert out.total_tokens == 64 and out.num_decode_tokens == 5 and out.num_prefill_tokens == 59
    out = run_step(s)                                         # the rows come with the next portion
    assert [(x.start, x.num_tokens) for x in out.scheduled][-1] == (59, 59) and out.total_tokens == 64
    # on a multiple already: 5 + 27 = 32 rows is under two tiles; 64 rows exactly stay
    s2, _ = make(pages=256, max_num_batched_tokens=256, long_prefill_token_threshold=64, step_row_multiple=32)
    s2.add_request(req(0, 200, max_tokens=4))
    assert [(x.start, x.num_tokens) for x in run_step(s2).scheduled] == [(0, 64)]
    # more than a quarter tile over: 64 + 9 decoding requests = 73 = 2 * 32 + 9 > 8
    s3, _ = make(pages=256, seqs=16, max_num_batched_tokens=256, long_prefill_token_threshold=64, step_row_multiple=32)
    for i in range(9):
        s3.add_request(req(i, 2, max_tokens=40))
    run_step(s3)
    s3.add_request(req(20, 300, max_tokens=4))
    out = run_step(s3)
    assert out.total_tokens == 73 and out.scheduled[-1].num_tokens == 64
    # the portion is the prompt's last: its request samples in this step and keeps its rows
    s4, _ = make(pages=256, max_num_batched_tokens=256, long_prefill_token_threshold=64, step_row_multiple=32)
    for i in range(5):
        s4.add_request(req(i, 3, max_tokens=40))
    run_step(s4)
    s4.add_request(req(9, 64, max_tokens=4))
    out = run_step(s4)
    assert out.total_tokens == 69 and out.scheduled[-1].want_logits


@pytest.mark.parametrize("seed", range(3))
def test_random_workloads_with_a_row_multiple_finish_too(seed):
    rng = random.Random(40 + seed)
    s, cache = make(pages=80, page=8, seqs=6, max_num_batched_tokens=96, long_prefill_token_threshold=40,
                    step_row_multiple=16, prefix=bool(seed % 2))
    todo = [req(i, rng.randint(1, 150), max_tokens=rng.randint(1, 30), first=1000 * (i % 3)) for i in range(16)]
    done, steps, cut = {}, 0, 0
    while todo or s.has_work():
        for _ in range(rng.randint(0, 2)):
            if todo:
                r = todo.pop(0)
                s.add_request(r)
                done[r.request_id] = r
        out = run_step(s)
        assert out.total_tokens <= 96 and len(s.running) <= 6
        cut += out.total_tokens >= 32 and out.total_tokens % 16 == 0
        steps += 1
        assert steps < 5000
    assert all(len(r.output_token_ids) == r.max_tokens for r in done.values()) and cut > 0
    assert cache.num_free_pages() == 80 and cache.usage()["free_slots"] == 6


def test_max_num_seqs():
    s, _ = make(seqs=2)
    for i in range(4):
        s.add_request(req(i, 5, max_tokens=2))
    out = run_step(s)
    assert [x.request.request_id for x in out.scheduled] == ["r0", "r1"]
    out = run_step(s)                     # both finish here (2 tokens each)
    out = run_step(s)
    assert [x.request.request_id for x in out.scheduled] == ["r2", "r3"]


def test_no_chunking_admits_whole_prompts_only():
    s, _ = make(max_num_batched_tokens=50, enable_chunked_prefill=False)
    s.add_request(req(0, 30)); s.add_request(req(1, 30))
    out = run_step(s)
    assert [(x.request.request_id, x.num_tokens) for x in out.scheduled] == [("r0", 30)]
    with pytest.raises(RequestRefused, match="chunked prefill"):
        s.add_request(req(2, 60))


def test_requests_that_can_never_fit_are_refused():
    s, _ = make(pages=4, max_model_len=100)
    with pytest.raises(RequestRefused, match="max_model_len"):
        s.add_request(req(0, 95, max_tokens=10))
    with pytest.raises(RequestRefused, match="more cache pages"):
        s.add_request(req(1, 60, max_tokens=10))
    with pytest.raises(RequestRefused, match="at least one"):
        s.add_request(req(2, 0))
    s.add_request(req(3, 50, max_tokens=14))
    with pytest.raises(RequestRefused, match="in use"):
        s.add_request(req(3, 5))


def test_waiting_request_is_not_admitted_without_pages():
    s, cache = make(pages=4)
    s.add_request(req(0, 40, max_tokens=20)); s.add_request(req(1, 40, max_tokens=20))
    out = run_step(s)
    assert [x.request.request_id for x in out.scheduled] == ["r0"] and not out.preempted
    assert cache.usage()["num_requests"] == 1          # the failed admission left nothing behind
    assert s.waiting[0].request_id == "r1"


def test_out_of_pages_preempts_the_newest_and_it_recomputes():
    s, cache = make(pages=4, page=16)
    s.add_request(req(0, 30, max_tokens=34)); s.add_request(req(1, 30, max_tokens=34))
    run_step(s)                                        # both prompts: 2 pages each, pool is full
    assert cache.num_free_pages() == 0
    out = run_step(s)                                  # token 31, 32: still inside page 2
    out = run_step(s)
    assert not out.preempted
    out = run_step(s)                                  # r0 needs a third page: r1, the newest, gives way
    assert out.preempted == ["r1"] and [x.request.request_id for x in out.scheduled] == ["r0"]
    r1 = s.requests["r1"]
    assert r1.status is RequestStatus.WAITING and r1.num_computed == 0 and len(r1.output_token_ids) == 3
    assert s.waiting[0] is r1 and s.num_preemptions == 1
    # r0 runs to its end; r1 comes back and computes prompt + generated again in one portion
    while "r0" in s.requests:
        out = run_step(s)
    out = run_step(s)
    back = [x for x in out.scheduled if x.request is r1]
    assert back and back[0].start == 0 and back[0].num_tokens == 33 and back[0].want_logits
    while s.has_work():
        run_step(s)
    assert len(r1.output_token_ids) == 34 and cache.num_free_pages() == 4


def test_a_lone_request_that_runs_out_preempts_itself_and_finishes_later():
    s, cache = make(pages=4, page=16)
    s.add_request(req(0, 20, max_tokens=30)); s.add_request(req(1, 20, max_tokens=30))
    steps = 0
    while s.has_work():
        run_step(s)
        steps += 1
        assert steps < 500
    assert s.num_preemptions >= 1 and cache.num_free_pages() == 4


def test_abort():
    s, cache = make()
    s.add_request(req(0, 20)); s.add_request(req(1, 20))
    run_step(s)
    assert s.abort_request("r0") and not s.abort_request("nobody")
    assert [r.request_id for r in s.running] == ["r1"] and cache.usage()["num_requests"] == 1
    s.add_request(req(2, 5))
    assert s.abort_request("r2") and not s.waiting


def test_prefix_hits_skip_computed_pages():
    s, cache = make(prefix=True, page=4, max_num_batched_tokens=100)
    s.add_request(Request("a", list(range(50, 68)), SamplingParams(max_tokens=2), 0, 0, 2))
    run_step(s); run_step(s)
    s.add_request(Request("b", list(range(50, 66)) + [1, 2, 3], SamplingParams(max_tokens=2), 1, 1, 2))
    out = run_step(s)
    assert [(x.start, x.num_tokens) for x in out.scheduled] == [(16, 3)] and s.prefix_hit_tokens == 16


def test_priority_policy_orders_the_waiting_queue_and_picks_the_victim():
    """crates/rllm-scheduler/src/policy.rs:16-95: larger priority first, arrival among equals; first come first
    served ignores the field.  A preempted request goes back to its place in that order, and the request that
    gives up its pages is the newest of the lowest priority."""
    def admitted(policy):
        s, _ = make(seqs=1, scheduling_policy=policy)
        for i, pr in enumerate([0, 5, 5, 9, -1]):
            r = req(i, 4, max_tokens=1)
            r.priority = pr
            s.add_request(r)
        order = []
        while s.has_work():
            out = run_step(s)
            order += [x.request.request_id for x in out.scheduled if x.start == 0]
        return order
    assert admitted("fcfs") == ["r0", "r1", "r2", "r3", "r4"]
    assert admitted("priority") == ["r3", "r1", "r2", "r0", "r4"]
    with pytest.raises(ValueError):
        make(scheduling_policy="lifo")
    # three requests of 16 tokens in a pool of four pages of 16: the first token that opens a page takes one from
    # the lowest priority, not from the newest
    s, cache = make(pages=4, page=16, seqs=4, scheduling_policy="priority")
    for i, pr in enumerate([1, 0, 2]):
        r = req(i, 16, max_tokens=20)
        r.priority = pr
        s.add_request(r)
    out = run_step(s)
    assert [x.request.request_id for x in out.scheduled] == ["r2", "r0", "r1"]        # admitted by priority
    out = run_step(s)                                       # each needs a second page: only one is free
    assert out.preempted == ["r1"] and [r.request_id for r in s.waiting] == ["r1"]
    s.add_request(req(7, 3, max_tokens=1))                  # priority 0, arrived later: behind r1 in the queue
    assert [r.request_id for r in s.waiting] == ["r1", "r7"]


def test_a_request_may_refuse_the_shared_pages():
    """crates/rllm-scheduler/src/scheduler.rs:565-580: ``skip_reading_prefix_cache`` computes the whole prompt."""
    s, cache = make(prefix=True)
    s.add_request(Request("a", list(range(50, 90)), SamplingParams(max_tokens=1), 0, 0, 1))
    run_step(s)
    s.add_request(Request("b", list(range(50, 90)) + [1], SamplingParams(max_tokens=1, skip_reading_prefix_cache=True), 1, 1, 1))
    s.add_request(Request("c", list(range(50, 90)) + [2], SamplingParams(max_tokens=1), 2, 2, 1))
    out = run_step(s)
    assert [(x.request.request_id, x.start, x.num_tokens) for x in out.scheduled] == [("b", 0, 41), ("c", 32, 9)]
    assert s.prefix_hit_tokens == 32


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_within_limits(seed):
    """Never more than max_num_seqs running or max_num_batched_tokens in a step;
    every request finishes; nothing is held at the end
    (crates/rllm-bench/tests/correctness.rs:247-326)."""
    rng = random.Random(seed)
    s, cache = make(pages=24, page=8, seqs=4, max_num_batched_tokens=48,
                    long_prefill_token_threshold=rng.choice([0, 16]))
    todo = [req(i, rng.randint(1, 90), max_tokens=rng.randint(1, 40)) for i in range(14)]
    done, steps = {}, 0
    while todo or s.has_work():
        for _ in range(rng.randint(0, 2)):
            if todo:
                r = todo.pop(0)
                s.add_request(r)
                done[r.request_id] = r
        out = run_step(s)
        assert out.total_tokens <= 48 and len(s.running) <= 4
        assert len({x.request.request_id for x in out.scheduled}) == len(out.scheduled)
        steps += 1
        assert steps < 5000
    assert all(len(r.output_token_ids) == r.max_tokens for r in done.values())
    assert cache.num_free_pages() == 24 and cache.usage()["free_slots"] == 4


def test_a_window_smaller_than_window_plus_portion_still_makes_progress():
    """A group that keeps a window of 24 keys, portions of 64 tokens and a pool of 4 pages of 16: the
    window fits (so the request is accepted), window plus portion does not.  The portion is cut to what
    fits, the window gives pages back on the way, and the request finishes without a preemption."""
    need = KVPagesNeed(2, 16, 24)
    cache = CacheManager([need], 16, 4, 4)
    s = Scheduler(SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, long_prefill_token_threshold=64,
                                  max_model_len=4096), cache)
    s.add_request(req(0, 200, max_tokens=40))
    s.add_request(req(1, 90, max_tokens=5))
    steps, sizes = 0, []
    while s.has_work():
        out = run_step(s)
        assert out.scheduled, "a step without tokens while requests wait: the loop would never end"
        sizes.append([x.num_tokens for x in out.scheduled])
        steps += 1
        assert steps < 400
    assert s.num_preemptions == 0
    assert sizes[0] == [64] and sizes[1] == [32]               # 4 pages, then what the window leaves free
    assert cache.num_free_pages() == 4 and cache.usage()["free_slots"] == 4


def test_max_tokens_is_what_ensure_takes():
    cache = CacheManager([KVPagesNeed(2, 16, None), KVPagesNeed(2, 16, 10)], 8, [6, 3], 2)
    cache.admit("a")
    assert cache.max_tokens("a", 0) == 24                        # the windowed pool: 3 pages of 8
    assert cache.ensure("a", 0, 24) and not cache.ensure("a", 24, 25 + 8)
    # queries from 24 on see keys 15..: pages 0 of the windowed group can go, one page comes free
    assert cache.max_tokens("a", 24) == 32
    assert cache.ensure("a", 24, 32) and cache.max_tokens("a", 32) == 40
    cache.free("a")
    cache.check()


def test_requests_that_arrive_together_share_a_prefix_that_only_one_computes():
    """Four requests with the same 48-token prefix arrive at once.  Pages become findable only after their
    keys exist, so the first is admitted alone; the others wait while it computes the common pages and are
    then admitted with hits: the prefix is computed once."""
    s, cache = make(prefix=True, page=16, pages=64, max_num_batched_tokens=32, long_prefill_token_threshold=0)
    shared = list(range(100, 148))
    for i in range(4):
        s.add_request(Request(f"r{i}", shared + [900 + 7 * i + j for j in range(10 + i)],
                              SamplingParams(max_tokens=3), i, i, 3))
    out = run_step(s)
    assert [(x.request.request_id, x.start, x.num_tokens) for x in out.scheduled] == [("r0", 0, 32)]
    out = run_step(s)                                  # r0's second portion: the third common page is still to come
    assert [x.request.request_id for x in out.scheduled] == ["r0"]
    out = run_step(s)                                  # the common pages exist: the others come in behind them
    got = {x.request.request_id: (x.start, x.num_tokens) for x in out.scheduled}
    assert got["r1"][0] == 48 and got["r2"][0] == 48 and s.prefix_hit_tokens >= 96
    while s.has_work():
        run_step(s)
    assert s.prefix_hit_tokens == 3 * 48 and cache.num_free_pages() == 64


def test_a_held_back_request_is_admitted_when_the_one_it_waits_for_goes_away():
    s, cache = make(prefix=True, page=16, pages=64, max_num_batched_tokens=16, long_prefill_token_threshold=0)
    shared = list(range(100, 148))
    s.add_request(Request("a", shared + [1, 2], SamplingParams(max_tokens=2), 0, 0, 2))
    s.add_request(Request("b", shared + [3, 4, 5], SamplingParams(max_tokens=2), 1, 1, 2))
    out = run_step(s)
    assert [x.request.request_id for x in out.scheduled] == ["a"]
    assert s.abort_request("a")
    out = run_step(s)                                  # nobody computes the prefix any more
    assert [(x.request.request_id, x.start) for x in out.scheduled] == [("b", 16)]     # a's first page had been registered
    while s.has_work():
        run_step(s)
    cache.check()


def test_a_portion_ends_at_the_pause_point_and_copies_go_on_from_there():
    """Several samples of one prompt: the first request stops before the prompt's last token, the others
    take its pages over (full pages shared, the partly filled one copied) and all compute the last
    token themselves."""
    s, cache = make(pages=16, max_num_batched_tokens=64)
    first = req(0, 41)
    first.pause_at = 40
    s.add_request(first)
    out = run_step(s)
    assert [(x.start, x.num_tokens, x.want_logits) for x in out.scheduled] == [(0, 40, False)]
    free_before = cache.num_free_pages()
    kids = []
    for i in (1, 2):
        kid = Request(("r0", i), first.prompt_token_ids, first.params, arrival=10 + i, seed=i, max_tokens=8)
        took = s.add_copy(first, kid)
        assert took is not None
        copies, (pslot, cslot) = took
        assert len(copies) == 1 and copies[0][0] == 0 and copies[0][1] == cache.table("r0", 0)[2]   # tokens 32..39 sit in page 2
        assert cslot != pslot and kid.status is RequestStatus.RUNNING and kid.num_computed == 40
        assert cache.table(kid.request_id, 0)[:2] == cache.table("r0", 0)[:2]
        assert cache.table(kid.request_id, 0)[2] == copies[0][2] != cache.table("r0", 0)[2]
        kids.append(kid)
    assert cache.num_free_pages() == free_before - 2 and s.num_copied_tokens == 80
    first.pause_at = None
    cache.check()
    out = run_step(s)
    assert [(x.request.request_id, x.start, x.num_tokens, x.want_logits) for x in out.scheduled] == \
        [("r0", 40, 1, True), (("r0", 1), 40, 1, True), (("r0", 2), 40, 1, True)]
    while s.has_work():
        run_step(s)
    assert cache.num_free_pages() == 16
    assert all(len(r.output_token_ids) == 8 for r in [first] + kids)


def test_a_copy_waits_like_a_new_request_when_nothing_can_be_taken_over():
    s, cache = make(pages=3, max_num_batched_tokens=64)
    first = req(0, 41, max_tokens=4)
    first.pause_at = 40
    s.add_request(first)
    run_step(s)                                   # 40 tokens: 3 pages, none left for a copy of the third
    kid = Request(("r0", 1), first.prompt_token_ids, first.params, arrival=11, seed=1, max_tokens=4)
    assert s.add_copy(first, kid) is None and kid.status is RequestStatus.WAITING and kid in s.waiting
    cache.check()
    other = Request(("r0", 2), first.prompt_token_ids, first.params, arrival=12, seed=2, max_tokens=4)
    assert s.add_copy(first, other, share=False) is None and other in s.waiting
    with pytest.raises(RequestRefused):
        s.add_copy(first, Request(("r0", 2), first.prompt_token_ids, first.params, arrival=13, seed=3, max_tokens=4))
    first.pause_at = None
    steps = 0
    while s.has_work():
        run_step(s)
        steps += 1
        assert steps < 200
    assert len(kid.output_token_ids) == 4 and len(other.output_token_ids) == 4 and cache.num_free_pages() == 3


@pytest.mark.parametrize("seed", range(8))
def test_everything_at_once_in_random_order(seed):
    """Priorities or first come first served, a row multiple, prefix sharing, a group with a window beside one
    that keeps every key, requests that pause before their last prompt token and hand copies on, aborts, few
    pages: every request that is not aborted finishes with its tokens, no step is empty while work waits,
    budgets hold, and nothing is held at the end."""
    rng = random.Random(900 + seed)
    windowed = seed % 2 == 1
    needs = [KVPagesNeed(2, 16, None)] + ([KVPagesNeed(1, 16, 24)] if windowed else [])
    pages = [40, 12] if windowed else [40]
    cache = CacheManager(needs, 8, pages, 6, enable_prefix_caching=seed % 4 < 2)
    budget = rng.choice([48, 96])
    s = Scheduler(SchedulerConfig(max_num_seqs=6, max_num_batched_tokens=budget, long_prefill_token_threshold=rng.choice([0, 24, 40]),
                                  max_model_len=4096, step_row_multiple=rng.choice([0, 16]),
                                  scheduling_policy=rng.choice(["fcfs", "priority"])), cache)
    todo = []
    for i in range(18):
        r = req(i, rng.randint(1, 120), max_tokens=rng.randint(1, 25), first=1000 * (i % 3))
        r.priority = rng.randint(-2, 2)
        if rng.random() < 0.3 and len(r.prompt_token_ids) > 1:
            r.pause_at = len(r.prompt_token_ids) - 1
        todo.append(r)
    live, aborted, copies, steps, arrivals = {}, set(), 0, 0, 100
    while todo or s.has_work():
        for _ in range(rng.randint(0, 2)):
            if todo:
                r = todo.pop(0)
                s.add_request(r)
                live[r.request_id] = r
        if live and rng.random() < 0.04:
            victim = rng.choice(sorted(live))
            if s.abort_request(victim):
                aborted.add(victim)
            live.pop(victim)
        had_work = s.has_work()
        out = run_step(s)
        assert out.total_tokens <= budget and len(s.running) <= 6
        assert len({x.request.request_id for x in out.scheduled}) == len(out.scheduled)
        if had_work and not out.scheduled:
            assert out.preempted or todo or not s.has_work() or s.running, "an empty step with nothing to wait for"
        for sc in out.scheduled:                                  # the engine's part: copies at the pause point
            r = sc.request
            if r.pause_at is not None and r.num_computed >= r.pause_at and r.status is RequestStatus.RUNNING:
                share = r.num_computed == r.pause_at
                r.pause_at = None
                arrivals += 1
                child = Request(f"{r.request_id}+", r.prompt_token_ids, r.params, arrivals, 7, r.max_tokens, priority=r.priority)
                s.add_copy(r, child, share)
                live[child.request_id] = child
                copies += 1
        for rid in [rid for rid, r in live.items() if r.status.finished]:
            live.pop(rid)
        steps += 1
        assert steps < 6000
    assert not live or all(r.status.finished for r in live.values())
    for g, n_all in enumerate(pages):
        assert cache.num_free_pages(g) == n_all
    assert cache.usage()["free_slots"] == 6
