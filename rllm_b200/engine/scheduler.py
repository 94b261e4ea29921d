"""Continuous batching: which requests run which tokens in the next step.

Each call of ``schedule`` (1) lets every running request go on, in order of
arrival: one token if it is decoding, the next portion of its prompt
otherwise; (2) admits waiting requests, first come first served (or, under the
``priority`` policy, larger ``Request.priority`` first and arrival among equals,
crates/rllm-scheduler/src/policy.rs:16-95), while the
token budget lasts, fewer than ``max_num_seqs`` run and a state slot is free.
A prompt is cut into portions under the step's token budget
(``max_num_batched_tokens``) and the portion cap
(``long_prefill_token_threshold``), anywhere, and continues over as many steps
as it needs.  A step that ends a few rows over a multiple of the products' row
tile gives those rows back (``step_row_multiple``, this engine's own).  This is the reference's order
(crates/rllm-scheduler/src/scheduler.rs:175-233; running :328-397, waiting
:402-532, budgets :480-495), except that there a prompt's later portions are
never scheduled as portions (:355-382) and a token is sampled after every
portion; here logits are asked for only when a portion ends at the last known
token.

With prefix sharing a waiting request whose prompt shares pages with a running
request that is still computing them is held back until they exist (the
reference picks the waiting request with the longest cached prefix,
:540-603, but registers pages after the compute like this engine, so requests
that arrive together would all compute their common prefix).

When pages run out: a waiting request is simply not admitted yet (:497-505).
A running request that needs a page and cannot get one makes room by
preemption (:357-375, :606-625): the newest running request (latest arrival; under
the priority policy the newest of the lowest priority) loses all its pages and
its slot and goes back into the waiting queue at its place in the queue's order; that is repeated until the page is there or the
request that asked is itself the newest, in which case it is the one
preempted.  A preempted request keeps its prompt and what it generated and
computes them again when readmitted; its samples are unchanged because its
random stream is indexed by the generated token.  A request that could never
fit (prompt plus ``max_tokens`` beyond ``max_model_len`` or beyond all pages)
is refused when it is added, so the loop cannot wait for ever.  Where a group
of layers keeps a window only, a request fits as soon as the window does; a
portion that would need more pages than are free (window plus portion) is cut
down to what fits instead of preempting the only request that could run.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from ..cache.manager import CacheManager, page_hashes
from ..sampling.params import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED_STOPPED = "stop"
    FINISHED_LENGTH = "length"
    FINISHED_ABORTED = "aborted"

    @property
    def finished(self) -> bool:
        return self.name.startswith("FINISHED")


class RequestRefused(ValueError):
    """A request that can never be served with this engine's limits."""


@dataclass
class Request:
    request_id: Hashable
    prompt_token_ids: List[int]
    params: SamplingParams
    arrival: int
    seed: int
    max_tokens: int
    output_token_ids: List[int] = field(default_factory=list)
    num_computed: int = 0            # tokens whose keys and values are in the cache
    num_cached_prefix: int = 0       # tokens taken over from shared pages at admission
    num_preemptions: int = 0
    status: RequestStatus = RequestStatus.WAITING
    prompt_page_hashes: Optional[List[bytes]] = None     # chained hashes of the prompt's full pages, made on demand
    family: Optional[Hashable] = None    # the id under which results are reported (several samples of one prompt share it)
    index: int = 0                       # which of the family's samples this is
    pause_at: Optional[int] = None       # a portion must end at this token, if it lies ahead: copies are taken there
    priority: int = 0                    # under the priority policy: larger values are admitted first

    @property
    def all_token_ids(self) -> List[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    def tokens(self, start: int, n: int) -> List[int]:
        """Tokens start .. start + n - 1 of prompt + generated, without joining the two lists."""
        p = len(self.prompt_token_ids)
        if start >= p:
            return self.output_token_ids[start - p:start - p + n]
        if start + n <= p:
            return self.prompt_token_ids[start:start + n]
        return self.prompt_token_ids[start:] + self.output_token_ids[:start + n - p]


@dataclass
class Scheduled:
    request: Request
    start: int
    num_tokens: int
    want_logits: bool


@dataclass
class SchedulerOutput:
    scheduled: List[Scheduled]
    preempted: List[Hashable]
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0

    @property
    def total_tokens(self) -> int:
        return sum(s.num_tokens for s in self.scheduled)


@dataclass
class SchedulerConfig:
    """Names of crates/rllm-core/src/config.rs:92-101."""

    max_num_seqs: int = 256
    max_num_batched_tokens: int = 4096
    long_prefill_token_threshold: int = 2048
    enable_chunked_prefill: bool = True
    max_model_len: int = 4096
    step_row_multiple: int = 0          # > 0: a step of many rows is cut down to a multiple of this many (see schedule)
    scheduling_policy: str = "fcfs"     # or "priority" (crates/rllm-core/src/config.rs:86-98)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager):
        if config.scheduling_policy not in ("fcfs", "priority"):
            raise ValueError(f"scheduling_policy must be fcfs or priority, not {config.scheduling_policy!r}")
        self.config = config
        self.cache = cache
        self.waiting: List[Request] = []
        self.running: List[Request] = []
        self.requests: Dict[Hashable, Request] = {}
        self.num_preemptions = 0
        self.prefix_hit_tokens = 0
        self.num_copied_tokens = 0          # tokens that requests took over from another by ``add_copy``
        self._windowed = any(getattr(cache.needs[g], "window", None) is not None for g in cache.paged)

    # ------------------------------------------------------------------
    def add_request(self, req: Request) -> None:
        if req.request_id in self.requests:
            raise RequestRefused(f"request id {req.request_id!r} is in use")
        if not req.prompt_token_ids:
            raise RequestRefused("a request needs at least one prompt token")
        most = len(req.prompt_token_ids) + req.max_tokens
        if most > self.config.max_model_len:
            raise RequestRefused(f"prompt ({len(req.prompt_token_ids)}) plus max_tokens ({req.max_tokens}) "
                                 f"exceeds max_model_len ({self.config.max_model_len})")
        if not self.cache.fits_at_all(most):
            raise RequestRefused(f"prompt plus max_tokens ({most} tokens) needs more cache pages than exist")
        if not self.config.enable_chunked_prefill and len(req.prompt_token_ids) > self.config.max_num_batched_tokens:
            raise RequestRefused("the prompt exceeds max_num_batched_tokens and chunked prefill is off")
        self.requests[req.request_id] = req
        self._enqueue(req)

    def _queue_key(self, req: Request):
        """The waiting queue's order: arrival, or priority (larger first) and then arrival
        (crates/rllm-scheduler/src/policy.rs:28-40, 88-95)."""
        return (-req.priority, req.arrival) if self.config.scheduling_policy == "priority" else (0, req.arrival)

    def _enqueue(self, req: Request) -> None:
        req.status = RequestStatus.WAITING
        i = 0
        while i < len(self.waiting) and self._queue_key(self.waiting[i]) < self._queue_key(req):
            i += 1
        self.waiting.insert(i, req)

    def add_copy(self, parent: Request, child: Request, share: bool = True):
        """``child`` goes on from where ``parent`` stands: it shares the pages that hold the parent's
        first ``num_computed`` tokens (a copy of a partly filled last page, a copy of the state slot) and
        runs from the next step on, without computing them again
        (crates/rllm-cache/src/manager.rs:220-245, which the reference's scheduler never calls).
        Returns what ``CacheStorage.copy_for_fork`` has to copy on the device before the next step.
        Where that cannot be (``share`` is off, the parent is not running or holds nothing yet, or a slot
        or a page is missing), the child waits like a new request and None is returned."""
        if child.request_id in self.requests:
            raise RequestRefused(f"request id {child.request_id!r} is in use")
        self.requests[child.request_id] = child
        took = None
        if (share and parent.status is RequestStatus.RUNNING and parent.num_computed > 0
                and len(self.running) < self.config.max_num_seqs):
            took = self.cache.fork(parent.request_id, child.request_id, parent.num_computed)
        if took is None:
            self._enqueue(child)
            return None
        child.num_computed = parent.num_computed
        self.num_copied_tokens += parent.num_computed
        child.status = RequestStatus.RUNNING
        self.running.append(child)
        self.running.sort(key=lambda r: r.arrival)
        return took

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------
    def _portion(self, req: Request, budget: int) -> int:
        left = req.num_tokens - req.num_computed
        n = min(left, budget)
        if left > 1 and self.config.long_prefill_token_threshold > 0:
            n = min(n, self.config.long_prefill_token_threshold)
        if req.pause_at is not None and req.num_computed < req.pause_at:
            n = min(n, req.pause_at - req.num_computed)
        return n

    def _prompt_hashes(self, req: Request) -> List[bytes]:
        if req.prompt_page_hashes is None:
            req.prompt_page_hashes = page_hashes(req.prompt_token_ids, self.cache.page_size)
        return req.prompt_page_hashes

    def _prefix_is_on_its_way(self, req: Request) -> bool:
        """With prefix sharing: whether a running request is still computing pages of its prompt that
        this waiting request's prompt shares and cannot find yet.  Admitting it now would compute the
        same pages twice (pages become findable only after their keys exist); a step or two later it
        finds them.  The running request makes progress whatever happens to this one, and if it is
        preempted or ends the test fails and the request is admitted as usual."""
        mine = self._prompt_hashes(req)
        if not mine or req.params.skip_reading_prefix_cache:
            return False
        page = self.cache.page_size
        have = self.cache.match_prefix(req.all_token_ids) // page
        for r in self.running:
            if r.num_computed >= len(r.prompt_token_ids):
                continue                              # its prompt's pages are all findable (or evicted: nothing to wait for)
            theirs = self._prompt_hashes(r)
            common = 0
            while common < len(mine) and common < len(theirs) and mine[common] == theirs[common]:
                common += 1
            if common > have and common > r.num_computed // page:
                return True
        return False

    def _preempt(self, req: Request, out: SchedulerOutput) -> None:
        self.cache.free(req.request_id)
        req.num_computed = 0
        req.num_cached_prefix = 0
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(req)
        self._enqueue(req)
        out.preempted.append(req.request_id)
        out.scheduled[:] = [s for s in out.scheduled if s.request is not req]

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput([], [])
        budget = self.config.max_num_batched_tokens
        # (1) running requests go on
        for req in list(self.running):
            if req.status is not RequestStatus.RUNNING:
                continue                      # preempted while an older request was scheduled
            if budget <= 0:
                break
            n = self._portion(req, budget)
            if n <= 0:
                continue
            if n < req.num_tokens - req.num_computed and not self.config.enable_chunked_prefill:
                continue
            # a decoding request needs a new page only when its next token opens one (and a window, if any
            # group has one, gives pages back on the way): skip the page bookkeeping otherwise
            if n == 1 and not self._windowed and req.num_computed % self.cache.page_size != 0:
                out.scheduled.append(Scheduled(req, req.num_computed, 1, req.num_computed + 1 == req.num_tokens))
                budget -= 1
                continue
            while not self.cache.ensure(req.request_id, req.num_computed, req.num_computed + n):
                victim = max(self.running, key=self._queue_key)      # the newest (of the lowest priority)
                if victim is req and n > 1:
                    # nobody newer to take pages from: a shorter portion may still fit (a window gives
                    # pages back on the way, so the rest follows in later steps)
                    fit = self.cache.max_tokens(req.request_id, req.num_computed) - req.num_computed
                    if fit >= 1:
                        n = min(n, fit)
                        continue
                self._preempt(victim, out)
                if victim is req:
                    break
            if req.status is not RequestStatus.RUNNING:
                continue
            out.scheduled.append(Scheduled(req, req.num_computed, n, req.num_computed + n == req.num_tokens))
            budget -= n
        # the budget of requests preempted after they were scheduled comes back
        budget = self.config.max_num_batched_tokens - out.total_tokens
        # (2) admit waiting requests, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.config.max_num_seqs \
                and self.cache.has_free_slot():
            req = self.waiting[0]
            if req.request_id in out.preempted:
                break                         # just preempted: not in the same step
            if self.cache.prefix_caching and self._prefix_is_on_its_way(req):
                break                         # first come, first served: those behind it wait too
            tokens = req.all_token_ids
            self.cache.admit(req.request_id)
            cached = 0 if req.params.skip_reading_prefix_cache else self.cache.adopt_prefix(req.request_id, tokens)
            req.num_computed = cached
            n = self._portion(req, budget)
            if not self.running and self.config.enable_chunked_prefill and n > 1:
                # the pools are empty and the portion still does not fit (a window plus the portion
                # needs more pages than the window alone): start with what fits
                fit = self.cache.max_tokens(req.request_id, req.num_computed) - req.num_computed
                if 1 <= fit < n:
                    n = fit
            whole = n == req.num_tokens - req.num_computed
            if (not whole and not self.config.enable_chunked_prefill) or \
                    not self.cache.ensure(req.request_id, req.num_computed, req.num_computed + n):
                self.cache.free(req.request_id)
                req.num_computed = 0
                break
            req.num_cached_prefix = cached
            self.prefix_hit_tokens += cached
            self.waiting.pop(0)
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            self.running.sort(key=lambda r: r.arrival)
            out.scheduled.append(Scheduled(req, req.num_computed, n, whole))
            budget -= n
        self._trim_to_row_multiple(out)
        for s in out.scheduled:
            if s.num_tokens == 1 and s.start >= len(s.request.prompt_token_ids):
                out.num_decode_tokens += 1
            else:
                out.num_prefill_tokens += s.num_tokens
        return out

    def _trim_to_row_multiple(self, out: SchedulerOutput) -> None:
        """The matrix products of a step work on tiles of ``step_row_multiple`` rows (128 for the tensor-core
        kernels), so a 512-token portion beside 15 decoding requests costs five row tiles where 512 rows cost
        four (measured on the products of a layer: 7 to 21 % more time for 3 % more tokens).  Where a step of
        at least two tiles ends up to a quarter tile over a multiple, the overhang is taken off a prompt
        portion that is not its prompt's last (its request samples nothing in this step either way, and the
        tokens come with its next portion).  The pages that were set aside for them stay with the request."""
        m = self.config.step_row_multiple
        total = out.total_tokens
        if m <= 0 or total < 2 * m:
            return
        over = total % m
        if over == 0 or over > m // 4:
            return
        for i in range(len(out.scheduled) - 1, -1, -1):
            s = out.scheduled[i]
            if not s.want_logits and s.num_tokens > over and s.start + s.num_tokens < s.request.num_tokens:
                out.scheduled[i] = Scheduled(s.request, s.start, s.num_tokens - over, False)
                return

    # ------------------------------------------------------------------
    def after_step(self, out: SchedulerOutput) -> None:
        """The step ran: its tokens' keys and values are in the cache."""
        for s in out.scheduled:
            req = s.request
            if req.status is not RequestStatus.RUNNING:
                continue                 # ended while the step was on the GPU: it holds nothing any more
            before = req.num_computed
            req.num_computed = s.start + s.num_tokens
            # content hashes only when a page was completed by this step
            if self.cache.prefix_caching and req.num_computed // self.cache.page_size > before // self.cache.page_size:
                self.cache.register_computed(req.request_id, req.all_token_ids, req.num_computed)

    def finish(self, req: Request, status: RequestStatus) -> None:
        """Take a request out and give back what it holds."""
        if req.status is RequestStatus.RUNNING:
            self.running.remove(req)
            self.cache.free(req.request_id)
        elif req.status is RequestStatus.WAITING:
            self.waiting.remove(req)
        req.status = status
        self.requests.pop(req.request_id, None)

    def abort_request(self, request_id: Hashable) -> bool:
        """crates/rllm-scheduler/src/scheduler.rs:165-171."""
        req = self.requests.get(request_id)
        if req is None:
            return False
        self.finish(req, RequestStatus.FINISHED_ABORTED)
        return True

    def stats(self) -> dict:
        """Fields of crates/rllm-scheduler/src/output.rs:51-64, plus prefix hits."""
        return {"num_running": len(self.running), "num_waiting": len(self.waiting),
                "num_preemptions": self.num_preemptions, "prefix_hit_tokens": self.prefix_hit_tokens,
                "num_copied_tokens": self.num_copied_tokens,
                "cache": self.cache.usage()}
