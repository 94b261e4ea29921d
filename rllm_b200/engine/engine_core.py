"""The engine: requests in, tokens out, one step at a time.

``step`` = schedule -> run the batch through the step function -> sample at
the rows whose portion ended at the last known token -> append the tokens ->
stop checks -> give finished requests' pages back
(crates/rllm-engine/src/engine_core.rs:91-226).  Stop checks, in the
reference's order (:153-163): an EOS token unless ``ignore_eos``, a token of
``stop_token_ids`` -> ``stop``; ``max_tokens`` generated -> ``length``; the
scheduler's limit ``max_model_len`` -> ``length``
(crates/rllm-scheduler/src/scheduler.rs:349-353).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional, Sequence

import torch

from ..cache import CacheManager, CacheStorage, page_bytes
from ..config.engine_args import EngineArgs
from ..models.decoder import DecoderModel
from ..parts.spec import KVPagesNeed
from .. import log
from ..sampling import Sampler, SamplingParams, SamplingRow
from .runner import ModelRunner, StepEntry
from .scheduler import Request, RequestRefused, RequestStatus, Scheduler, SchedulerConfig, SchedulerOutput


@dataclass
class Usage:
    """crates/rllm-core/src/output.rs:29-34."""

    prompt_tokens: int
    completion_tokens: int
    total_tokens: int


@dataclass
class Logprob:
    """crates/rllm-core/src/output.rs:44-49 (no text), with the likeliest tokens of the place beside it
    (crates/rllm-sampling/src/sampler.rs:27-31)."""

    token_id: int
    logprob: float
    top_logprobs: List[tuple] = field(default_factory=list)      # (token id, log-probability), descending


@dataclass
class CompletionOutput:
    """crates/rllm-core/src/output.rs:13-20 (no text: the engine works on ids)."""

    index: int
    token_ids: List[int]
    finish_reason: Optional[str] = None      # "stop" | "length" | "aborted"
    logprobs: Optional[List[Logprob]] = None # one for each token of token_ids, if the request asked for them


@dataclass
class RequestOutput:
    """crates/rllm-core/src/output.rs:6-11, plus the prompt for convenience."""

    request_id: Hashable
    prompt_token_ids: List[int]
    outputs: List[CompletionOutput]
    finished: bool
    usage: Usage


def plan_cache_pages(model: DecoderModel, args: EngineArgs, max_model_len: int, device: torch.device) -> List[int]:
    """Pages of every paged group of layers, in the order of the groups.

    A group that keeps all keys can use max_num_seqs * ceil(max_model_len / block_size) pages, the
    reference's sizing rule (crates/rllm-server/src/server.rs:367-370).  A group that keeps a window
    holds, per request, the window plus the portion being computed, so it is given
    ceil((window + portion) / block_size) + 1 pages a request and never more than the rule above.
    ``num_gpu_blocks``, if given, is the count of the all-keys groups (windowed groups take no more than
    they can use).  Otherwise the counts come from memory, as the reference's unused formula intends
    (crates/rllm-cache/src/spec.rs:45-60: available bytes / bytes of a page over all layers): what
    ``gpu_memory_utilization`` of the device leaves beside the weights and a reserve for activations
    is shared so that every group gets the same fraction of what it can use."""
    bs = args.block_size
    elem = 2 if model.dtype is torch.bfloat16 else 4
    portion = args.max_num_batched_tokens
    if args.long_prefill_token_threshold > 0:
        portion = min(portion, args.long_prefill_token_threshold)
    full = -(-max_model_len // bs)
    useful, nbytes = [], []
    for g, need in enumerate(model.layout.groups):
        if not isinstance(need, KVPagesNeed):
            continue
        per_request = full if need.window is None else min(full, -(-(need.window + portion) // bs) + 1)
        useful.append(args.max_num_seqs * per_request)
        nbytes.append(page_bytes(need, bs, elem) * len(model.layout.owners[g]))
    if not useful:
        return []
    if args.num_gpu_blocks is not None:
        return [min(args.num_gpu_blocks, u) if need_windowed else args.num_gpu_blocks
                for u, need_windowed in zip(useful, _windowed(model))]
    torch.cuda.empty_cache()          # blocks that PyTorch's allocator holds but nobody uses (the loader's temporaries) are free
    free, total = torch.cuda.mem_get_info(device)
    spec = model.spec
    act = args.max_num_batched_tokens * (spec.hidden_size * 16 + 64 * 1024) + \
        min(args.max_num_seqs, args.max_num_batched_tokens) * spec.vocab_size * 8 + (1 << 30)
    budget = int(total * args.gpu_memory_utilization) - (total - free) - act
    if budget < 4 * sum(nbytes):
        raise RuntimeError(f"no room for a KV cache: {free >> 20} MiB free of {total >> 20} MiB with "
                           f"gpu_memory_utilization {args.gpu_memory_utilization}")
    share = min(1.0, budget / sum(u * b for u, b in zip(useful, nbytes)))
    return [max(4, int(u * share)) for u in useful]


def _windowed(model: DecoderModel) -> List[bool]:
    return [need.window is not None for need in model.layout.groups if isinstance(need, KVPagesNeed)]


@dataclass(frozen=True)
class SampleId:
    """The scheduler's and the cache's name of sample ``index`` > 0 of request ``request``."""

    request: Hashable
    index: int


@dataclass
class _Family:
    """The samples of a request with ``n`` > 1: ``members`` as far as they exist yet."""

    n: int
    members: List[Request]
    unfinished: int
    spread: bool = False           # the samples beyond the first have been made


class EngineCore:
    ERROR_POLL_STEPS = 8           # the kernels' error words are looked at every this many steps

    def __init__(self, model: DecoderModel, args: Optional[EngineArgs] = None):
        self.args = args or EngineArgs()
        self.args.validate()
        self.model = model
        self.device = model.device
        spec = model.spec
        self.max_model_len = min(self.args.max_model_len or spec.max_positions, spec.max_positions)
        pages = plan_cache_pages(model, self.args, self.max_model_len, self.device)
        self.num_pages = list(pages)
        self.cache = CacheManager(model.layout.groups, self.args.block_size, pages,
                                  self.args.max_num_seqs, self.args.enable_prefix_caching)
        self.storage = CacheStorage(model.layout, self.args.block_size, pages,
                                    self.args.max_num_seqs, model.dtype, self.device)
        self.runner = ModelRunner(model, self.cache, self.storage, self.args.enable_cuda_graphs)
        self.sampler = Sampler(self.device)
        self.scheduler = Scheduler(SchedulerConfig(
            max_num_seqs=self.args.max_num_seqs, max_num_batched_tokens=self.args.max_num_batched_tokens,
            long_prefill_token_threshold=self.args.long_prefill_token_threshold,
            enable_chunked_prefill=self.args.enable_chunked_prefill, max_model_len=self.max_model_len,
            step_row_multiple=self.args.step_row_multiple, scheduling_policy=self.args.scheduling_policy),
            self.cache)
        self.eos_token_ids = tuple(spec.eos_token_ids)
        self._arrivals = itertools.count()
        self.num_steps = 0
        self._prepared = None          # (schedule, requests, plain_greedy, graph) of the next step, made ahead
        self._inflight = None          # (schedule, requests, plain_greedy, sampled, read-back) of a step already on the GPU
        self._readback = [None, None]  # pinned buffers and events for the sampled tokens, used in turn
        self._readback_next = 0
        self.num_steps_ahead = 0       # steps that were put on the GPU before the tokens of the step before were read
        self.last_schedule: Optional[SchedulerOutput] = None
        self._families: Dict[Hashable, _Family] = {}      # requests with n > 1, by their id

    # ------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None, priority: int = 0) -> Hashable:
        """crates/rllm-engine/src/engine_core.rs:55-80.  ``priority`` counts under the priority policy only
        (crates/rllm-core/src/request.rs:136)."""
        params = params or SamplingParams()
        params.validate()
        arrival = next(self._arrivals)
        rid = request_id if request_id is not None else arrival
        vocab = self.model.spec.vocab_size
        prompt = [int(t) for t in prompt_token_ids]
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"request {rid!r}: a prompt token lies outside the vocabulary of {vocab}")
        max_tokens = params.max_tokens if params.max_tokens is not None else self.max_model_len - len(prompt)
        seed = params.seed if params.seed is not None else (self.args.seed * 1000003 + arrival)
        if rid in self._families:
            raise RequestRefused(f"request id {rid!r} is in use")
        req = Request(rid, prompt, params, arrival, seed, max_tokens, family=rid, priority=int(priority))
        self.scheduler.add_request(req)
        self._prepared = None          # a step prepared ahead did not know of this request
        if params.n > 1:
            fam = self._families[rid] = _Family(params.n, [req], params.n)
            if len(prompt) > 1 and self.args.enable_chunked_prefill:
                req.pause_at = len(prompt) - 1       # the other samples branch off before the prompt's last token
            else:
                self._spread(fam)
        return rid

    def _spread(self, fam: _Family) -> None:
        """Make samples 1 .. n-1 of a request.  The first sample has computed all of the prompt but its
        last token: the others take that over (shared pages, a copy of the last, partly filled page and
        of the state slot) and every sample computes the last token itself, so that a mixer's state
        branches at the right place and no row of logits has to serve twice.  Each sample has a random
        stream of its own: its seed is the request's seed moved on by the sample's index.  Where nothing
        can be taken over (a prompt of one token, prompts that run whole, no slot or page free right
        now) the samples wait like new requests with the same prompt."""
        first = fam.members[0]
        fam.spread = True
        # (a prompt whose pages were all found in the cache starts at the branching point and has passed it)
        share = first.pause_at is not None and first.num_computed == first.pause_at
        first.pause_at = None
        for i in range(1, fam.n):
            seed = (first.seed + i * 0x9E3779B97F4A7C15) & 0x7FFFFFFFFFFFFFFF
            child = Request(SampleId(first.request_id, i), first.prompt_token_ids, first.params,
                            next(self._arrivals), seed, first.max_tokens, family=first.request_id, index=i,
                            priority=first.priority)
            took = self.scheduler.add_copy(first, child, share)
            if took is not None:
                with torch.cuda.device(self.device):
                    self.storage.copy_for_fork(*took)
            fam.members.append(child)
        self._prepared = None

    def abort_request(self, request_id: Hashable) -> bool:
        self._prepared = None
        fam = self._families.pop(request_id, None)
        if fam is None:
            return self.scheduler.abort_request(request_id)
        found = [self.scheduler.abort_request(r.request_id) for r in fam.members]
        return any(found)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------
    def step(self) -> List[RequestOutput]:
        with log.span("engine_step"):
            return self._step()

    def _step(self) -> List[RequestOutput]:
        inflight, self._inflight = self._inflight, None
        prepared, self._prepared = self._prepared, None
        if inflight is not None and not any(r.status is RequestStatus.RUNNING for r in inflight[1]):
            inflight = None            # every request of the step in flight has ended: nothing of it is wanted
        if inflight is not None:
            # this step was put on the GPU during the last call, behind the step before it
            sched, sampled_reqs, plain_greedy, sampled, pending = inflight
            wanted_lp = None               # a request that wants log-probabilities is never launched ahead
            self.last_schedule = sched
        elif prepared is not None:
            # the schedule and the packed inputs of this step were made while the GPU ran the last one
            sched, sampled_reqs, plain_greedy, graph = prepared
            self.last_schedule = sched
            self.num_steps += 1
            logits = self.runner.run_prepared(graph)
            raw = self._raw_logits(logits, sampled_reqs)
            sampled = self._sample(logits, sampled_reqs, plain_greedy, 0)
            wanted_lp = self._logprobs(raw, sampled, sampled_reqs)
            pending = self._read_back(sampled, graph)
        else:
            with log.span("schedule"):
                sched = self.scheduler.schedule()
            self.last_schedule = sched
            self.num_steps += 1
            if not sched.scheduled:
                if not sched.preempted and not self.scheduler.running and self.scheduler.waiting:
                    # nothing runs, nothing was preempted and still nobody could be admitted: no later
                    # call would do better, and a caller that loops on has_work() would never return
                    raise RuntimeError("the scheduler cannot admit any waiting request although nothing is "
                                       f"running (cache: {self.cache.usage()})")
                return []
            entries, sampled_reqs = [], []
            plain_greedy = True            # every sampled row: argmax of untouched logits
            for s in sched.scheduled:
                req = s.request
                toks = req.tokens(s.start, s.num_tokens)
                entries.append(StepEntry(req.request_id, toks, s.start, [s.num_tokens - 1] if s.want_logits else []))
                if s.want_logits:
                    sampled_reqs.append(req)
                    p = req.params
                    plain_greedy = plain_greedy and p.greedy and not p.edits_logits
            with log.span("model_forward"):
                logits = self.runner.step(entries)
            raw = self._raw_logits(logits, sampled_reqs)
            with log.span("sampling"):
                sampled = self._sample(logits, sampled_reqs, plain_greedy, 0)
            wanted_lp = self._logprobs(raw, sampled, sampled_reqs)
            pending = self._read_back(sampled)
        # requests that ended (or were aborted) after this step went to the GPU: their rows are dropped
        live = [r.status is RequestStatus.RUNNING for r in sampled_reqs]
        # The GPU is busy now.  What does not depend on the sampled tokens is done meanwhile: the
        # bookkeeping of this step and, if the next step is sure to be a plain decode step of the same
        # requests, its schedule and its packed inputs; and that step is launched at once, behind this
        # one, with this step's tokens as its input on the device, unless a request wants its logits
        # edited by what it has generated.
        self.scheduler.after_step(sched)
        if self._families:
            for s in sched.scheduled:
                r = s.request
                if r.pause_at is not None and r.num_computed >= r.pause_at and r.status is RequestStatus.RUNNING:
                    self._spread(self._families[r.family])
        nxt = self._prepare_next(sched, sampled_reqs, plain_greedy) if all(live) else None
        if nxt is not None and self._launch_ahead(nxt, sampled_reqs, sampled):
            nxt = None
        tokens = self._tokens_of(pending)
        # the kernels' error words are read without waiting for the GPU, every few steps (two small copies in
        # the stream each time): a bad index shows a few steps late, and at the latest when generation ends
        if self.num_steps % self.ERROR_POLL_STEPS == 0:
            self.runner.poll_errors()
        outputs = []
        any_finished = False
        lps = self._logprobs_of(wanted_lp, sampled_reqs, tokens)
        for row, (req, tok, alive) in enumerate(zip(sampled_reqs, tokens, live)):
            if not alive:
                continue
            req.output_token_ids.append(int(tok))
            reason = self._finish_reason(req, int(tok))
            if reason is not None:
                any_finished = True
                self.scheduler.finish(req, RequestStatus.FINISHED_STOPPED if reason == "stop"
                                      else RequestStatus.FINISHED_LENGTH)
            n_prompt, n_out = len(req.prompt_token_ids), len(req.output_token_ids)
            done = reason is not None
            fam = self._families.get(req.family)
            if fam is not None:
                # several samples of one prompt: reported under the request's id, finished with the last of them
                n_out = sum(len(r.output_token_ids) for r in fam.members)
                if done:
                    fam.unfinished -= 1
                    done = fam.unfinished == 0
                    if done:
                        del self._families[req.family]
            outputs.append(RequestOutput(req.family, req.prompt_token_ids,
                                         [CompletionOutput(req.index, [int(tok)], reason, lps.get(row))], done,
                                         Usage(n_prompt, n_out, n_prompt + n_out)))
        if log.logger.isEnabledFor(log.logging.DEBUG):
            log.logger.debug("step %d: %d prompt + %d decode tokens, %d sampled, %d finished, %d preempted; "
                             "running %d waiting %d free pages %d", self.num_steps, sched.num_prefill_tokens,
                             sched.num_decode_tokens, len(sampled_reqs), sum(o.finished for o in outputs),
                             len(sched.preempted), len(self.scheduler.running), len(self.scheduler.waiting),
                             self.cache.num_free_pages())
        if nxt is not None and not any_finished and not self.scheduler.waiting:
            by_req = {r.request_id: t for r, t in zip(sampled_reqs, tokens)}
            nxt[3].patch_tokens([by_req[s.request.request_id] for s in nxt[0].scheduled])
            self._prepared = nxt
        return outputs

    def _read_back(self, sampled, graph=None):
        """Start the copy of a step's sampled tokens to pinned host memory, right behind the sampling
        kernel in the stream; returns what ``_tokens_of`` waits for.  A plain ``tolist`` would wait for
        everything queued since, a step launched ahead included.  With the decode graph that ran the
        step, one kernel writes the tokens to the host and makes them the graph's next input."""
        if sampled is None:
            return None
        n = sampled.numel()
        slot = self._readback[self._readback_next]
        self._readback_next ^= 1
        if slot is None or slot[0].numel() < n:
            slot = (torch.empty(max(n, self.args.max_num_seqs), dtype=torch.int32, pin_memory=True), torch.cuda.Event())
            self._readback[self._readback_next ^ 1] = slot
        with torch.cuda.device(self.device):
            if graph is not None:
                graph.advance(sampled, slot[0])
            else:
                slot[0][:n].copy_(sampled, non_blocking=True)
            slot[1].record()
        return slot[0], slot[1], n

    @staticmethod
    def _tokens_of(pending) -> List[int]:
        if pending is None:
            return []
        buf, event, n = pending
        event.synchronize()
        return buf[:n].tolist()

    def _sample(self, logits, sampled_reqs, plain_greedy: bool, ahead: int):
        """The next tokens int32 [R] on the device; ``ahead``: tokens that the requests will have
        generated by then beyond those the host knows (1 for a step launched ahead)."""
        if not sampled_reqs:
            return None
        if plain_greedy:
            return self.sampler.greedy(logits)
        rows = [SamplingRow(r.params, r.seed, len(r.output_token_ids) + ahead,
                            r.all_token_ids if r.params.edits_logits else (), self.eos_token_ids)
                for r in sampled_reqs]
        return self.sampler.sample(logits, rows)

    def _raw_logits(self, logits, sampled_reqs):
        """A copy of the step's logits before anything edits them, if a request wants log-probabilities
        (they are taken from the raw logits, crates/rllm-sampling/src/sampler.rs:149-160), else None."""
        if not any(r.params.logprobs is not None for r in sampled_reqs):
            return None
        return logits.clone()

    def _logprobs(self, raw, sampled, sampled_reqs):
        """Device tensors (lp, top ids, top values) for the rows of the step, or None."""
        if raw is None or sampled is None:
            return None
        from ..kernels import ops
        top_n = max(r.params.logprobs or 0 for r in sampled_reqs)
        with torch.cuda.device(self.device):
            return ops.logprobs(raw, sampled, top_n)

    @staticmethod
    def _logprobs_of(wanted_lp, sampled_reqs, tokens) -> Dict[int, List[Logprob]]:
        """row -> [Logprob] for the rows whose request asked for log-probabilities."""
        if wanted_lp is None:
            return {}
        lp, ids, vals = (t.cpu() for t in wanted_lp)
        out = {}
        for row, req in enumerate(sampled_reqs):
            n = req.params.logprobs
            if n is None:
                continue
            top = [(int(i), float(v)) for i, v in zip(ids[row, :n].tolist(), vals[row, :n].tolist()) if i >= 0]
            out[row] = [Logprob(int(tokens[row]), float(lp[row]), top)]
        return out

    def _launch_ahead(self, nxt, sampled_reqs, sampled) -> bool:
        """Put the prepared next step on the GPU now.  Its rows are the same requests in the same order,
        so the tokens being sampled are copied into its input on the device.  If one of the requests
        turns out to end on this step's token, its row of the step in flight is computed for nothing and
        dropped; the others' rows do not depend on it."""
        nsched, nreqs, plain_greedy, graph = nxt
        if sampled is None or len(nreqs) != len(sampled_reqs) or any(a is not b for a, b in zip(nreqs, sampled_reqs)):
            return False
        if any(r.params.edits_logits or r.params.logprobs is not None for r in nreqs):
            return False
        self.num_steps += 1
        self.num_steps_ahead += 1
        with torch.cuda.device(self.device), torch.no_grad():
            if graph.commit():
                graph.token_ids[: sampled.numel()].copy_(sampled, non_blocking=True)
            logits = graph.run()
        ahead = self._sample(logits, nreqs, plain_greedy, 1)
        self._inflight = (nsched, nreqs, plain_greedy, ahead, self._read_back(ahead, graph))
        return True

    def _prepare_next(self, sched: SchedulerOutput, sampled_reqs, plain_greedy):
        """Schedule and pack the next step ahead of time, if it is certain to be a decode step of exactly
        the requests that were just sampled (unless one of them stops on the token being sampled, which
        the caller finds out).  Returns (schedule, requests, plain_greedy, graph) or None."""
        sch = self.scheduler
        if (not self.args.enable_cuda_graphs or sch.waiting or not sampled_reqs
                or len(sampled_reqs) != len(sched.scheduled) or len(sampled_reqs) != len(sch.running)
                or self.cache.num_free_pages() < len(sampled_reqs)):
            return None
        for s in sched.scheduled:
            r = s.request
            if (s.num_tokens != 1 or len(r.output_token_ids) + 2 > r.max_tokens
                    or r.num_tokens + 2 > self.max_model_len):
                return None
        for r in sampled_reqs:
            r.output_token_ids.append(-1)          # stands for the token being sampled right now
        try:
            nsched = sch.schedule()
            ok = (not nsched.preempted and len(nsched.scheduled) == len(sampled_reqs)
                  and all(s.num_tokens == 1 and s.want_logits for s in nsched.scheduled))
            graph = None
            if ok:
                entries = [StepEntry(s.request.request_id, [0], s.start, [0]) for s in nsched.scheduled]
                graph = self.runner.prepare_decode(entries)
        finally:
            for r in sampled_reqs:
                r.output_token_ids.pop()
        if graph is None:
            return None
        return nsched, [s.request for s in nsched.scheduled], plain_greedy, graph

    def _finish_reason(self, req: Request, token: int) -> Optional[str]:
        p = req.params
        if (token in self.eos_token_ids and not p.ignore_eos) or token in p.stop_token_ids:
            return "stop"
        if len(req.output_token_ids) >= req.max_tokens:
            return "length"
        if req.num_tokens >= self.max_model_len:
            return "length"
        return None

    def stats(self) -> dict:
        return dict(self.scheduler.stats(), num_steps=self.num_steps, num_steps_ahead=self.num_steps_ahead)
