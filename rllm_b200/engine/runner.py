"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step(entries)`` takes any mix of prompt portions and single
decoded tokens, cut anywhere.  It runs exactly the tokens it is given, as one
flat batch, against the cache that earlier steps left, writes their keys and
values (and states) into the cache, and returns float32 logits at the places
that were asked for, in the order of the entries and of each entry's ``want``.
It does no request bookkeeping: the caller (scheduler or replay) owns
positions and pages.

The reference's counterpart builds its flat batch in
crates/rllm-worker/src/model_runner.rs:136-256 (prefills first, then decodes,
positions from ``num_computed``; slot rule :806-826) and its attention metadata
at :262-344; its executor computes logits for every row and keeps one per
sequence (crates/rllm-executor/src/uniproc.rs:167-175).  Here a decode is just
a portion of length 1, sequences with one token are placed first so that the
decode attention kernel sees a contiguous range, and the head runs on the
wanted rows only.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..models.decoder import DecoderModel
from ..parts.base import StepContext


class StepError(RuntimeError):
    pass


@dataclass
class StepEntry:
    req: Hashable
    tokens: Sequence[int]
    start: int                       # position of tokens[0] in its sequence
    want: Sequence[int] = ()         # indices into ``tokens`` whose logits are asked for


_ERR_BITS = {1: "a token id outside the vocabulary", 2: "a cache write to a page the request does not hold",
             4: "an attention read from a page the request does not hold"}


class BatchBuilder:
    """Flattens entries into the device arrays of a ``StepContext``."""

    def __init__(self, cache: CacheManager, device: torch.device, act_dtype: torch.dtype):
        if device.type != "cuda":
            raise StepError("the engine runs on a CUDA device only; there is no CPU path")
        self.cache, self.device, self.act_dtype = cache, device, act_dtype
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        # ring of pinned staging buffers; a buffer is reused only after its copy has run
        self._ring: List[list] = [[None, None] for _ in range(4)]
        self._ring_next = 0

    # ------------------------------------------------------------------
    def _stage(self, n: int):
        slot = self._ring[self._ring_next]
        self._ring_next = (self._ring_next + 1) % len(self._ring)
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0] is None or slot[0].numel() < n:
            slot[0] = torch.empty(max(n, 1 << 16), dtype=torch.int32, pin_memory=True)
        if slot[1] is None:
            slot[1] = torch.cuda.Event()
        return slot[0][:n], slot[1]

    def build_context(self, entries: Sequence[StepEntry]):
        """Flatten the entries: (StepContext, token ids, logit rows)."""
        for e in entries:
            if len(e.tokens) == 0:
                raise StepError(f"request {e.req!r}: an entry needs at least one token")
            if e.start < 0:
                raise StepError(f"request {e.req!r}: negative position")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"request {e.req!r}: wanted place {w} outside its {len(e.tokens)} tokens")
        if len({e.req for e in entries}) != len(entries):
            raise StepError("a request appears twice in one step")
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
        num_decode = sum(1 for e in entries if len(e.tokens) == 1)
        S = len(entries)
        q_lens = [len(entries[i].tokens) for i in order]
        T = sum(q_lens)
        q_start = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        first_of = {order[s]: int(q_start[s]) for s in range(S)}     # entry index -> first flat token
        token_ids = np.empty(T, dtype=np.int32)
        positions = np.empty(T, dtype=np.int32)
        token_seq = np.empty(T, dtype=np.int32)
        seq_lens = np.empty(S, dtype=np.int32)
        slots = np.empty(S, dtype=np.int32)
        paged = self.cache.paged
        tables = []
        for s, i in enumerate(order):
            e = entries[i]
            a, b = q_start[s], q_start[s + 1]
            token_ids[a:b] = np.asarray(e.tokens, dtype=np.int64)
            positions[a:b] = np.arange(e.start, e.start + (b - a), dtype=np.int32)
            token_seq[a:b] = s
            seq_lens[s] = e.start + (b - a)
            slots[s] = self.cache.slot(e.req)
        rows = np.asarray([first_of[i] + w for i, e in enumerate(entries) for w in e.want], dtype=np.int32)
        reqs = [entries[i].req for i in order]
        need = [-(-int(seq_lens[s]) // self.cache.page_size) for s in range(S)]
        width = max(1, max(need))
        for g in paged:
            for s, n in enumerate(need):
                have = self.cache.table_len(reqs[s], g)
                if have < n:
                    raise StepError(f"request {reqs[s]!r} holds {have} pages of group {g}, "
                                    f"its {int(seq_lens[s])} tokens need {n}")
            tab = np.empty((S, width), dtype=np.int32)
            self.cache.pack_tables(reqs, g, tab)
            for s, n in enumerate(need):
                tab[s, n:] = -1                     # pages behind this step's tokens are not this step's business
            tables.append(tab)
        # one pinned staging buffer, one copy to the device
        parts = [token_ids, positions, token_seq, q_start, seq_lens, slots, rows] + [t.ravel() for t in tables]
        sizes = [p.size for p in parts]
        total = sum(sizes)
        stage, copied = self._stage(total)
        host = stage.numpy()
        off = 0
        for p, n in zip(parts, sizes):
            host[off:off + n] = p
            off += n
        dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(stage, non_blocking=True)
        copied.record()
        views, off = [], 0
        for n in sizes:
            views.append(dev[off:off + n])
            off += n
        d_tokens, d_pos, d_tseq, d_qstart, d_seqlens, d_slots, d_rows = views[:7]
        block_tables: List[Optional[torch.Tensor]] = [None] * len(self.cache.needs)
        for g, tab, v in zip(paged, tables, views[7:]):
            block_tables[g] = v.view(tab.shape)
        ctx = StepContext(
            num_tokens=T, num_seqs=S, num_decode=num_decode, positions=d_pos, token_seq=d_tseq,
            q_start=d_qstart, seq_lens=d_seqlens, q_lens_host=q_lens,
            seq_lens_host=[int(x) for x in seq_lens], block_tables=block_tables, state_slots=d_slots,
            state_slots_host=[int(x) for x in slots], err=self.err, act_dtype=self.act_dtype)
        ctx.extras["starts_host"] = [entries[i].start for i in order]
        return ctx, d_tokens, d_rows


class ModelRunner:
    MAX_GRAPHS = 96

    def __init__(self, model: DecoderModel, cache: CacheManager, storage: CacheStorage,
                 enable_cuda_graphs: bool = True):
        if model.device is None:
            raise StepError("the model has no weights yet")
        self.model, self.cache, self.storage = model, cache, storage
        self.device = model.device
        self.builder = BatchBuilder(cache, self.device, model.dtype)
        self.err = self.builder.err
        # decode steps go through CUDA graphs if every part of every block says its forward can be captured
        self.capture_graphs = bool(enable_cuda_graphs) and all(
            getattr(p, "graph_safe", False) for b in model.blocks for p in b.parts())
        self.graphs = {}
        self.graph_pool = None

    def _decode_graph(self, entries: Sequence[StepEntry], pad: bool = True):
        from .decode_graph import DecodeGraph, batch_bucket, table_width_bucket
        page = self.cache.page_size
        blocks = max(-(-(e.start + 1) // page) for e in entries)
        # padding rows live on the storage's spare page and spare state slot
        key = (batch_bucket(len(entries)) if pad else len(entries), table_width_bucket(blocks))
        g = self.graphs.get(key)
        if g is None:
            if len(self.graphs) >= self.MAX_GRAPHS:
                return None
            if self.graph_pool is None:
                self.graph_pool = torch.cuda.graph_pool_handle()
            g = self.graphs[key] = DecodeGraph(self, *key)
        return g

    def build_context(self, entries: Sequence[StepEntry]):
        return self.builder.build_context(entries)

    # ------------------------------------------------------------------
    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Logits float32 [sum of len(want), vocab] on the device."""
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            self.storage.zero_slots(self.cache.take_fresh_slots())
            if self.capture_graphs and all(len(e.tokens) == 1 for e in entries):
                g = self._decode_graph(entries)
                if g is not None:
                    g.fill(entries)
                    logits = g.run()
                    wanted = [s for s, e in enumerate(entries) if len(e.want)]
                    if len(wanted) == len(entries):
                        return logits
                    return logits[torch.tensor(wanted, dtype=torch.long, device=self.device)]
            ctx, token_ids, rows = self.build_context(entries)
            return self.model.forward(token_ids, ctx, rows, self.storage)

    def prepare_decode(self, entries: Sequence[StepEntry]):
        """Get the next decode step ready on the host while the GPU is still busy with the current one:
        picks the captured graph of this shape and packs the inputs into its pinned buffer.  Returns the
        graph (to be given to ``run_prepared``, after ``patch_tokens`` if the tokens were not known yet),
        or None if this step cannot go through an already captured graph."""
        if not self.capture_graphs or not entries or any(len(e.tokens) != 1 or len(e.want) != 1 for e in entries):
            return None
        if self.cache.fresh_slots:
            return None
        g = self._decode_graph(entries)
        if g is None or g.graph is None:
            return None
        g.fill_host(entries)
        return g

    @torch.no_grad()
    def run_prepared(self, g) -> torch.Tensor:
        with torch.cuda.device(self.device):
            g.commit()
            return g.run()

    @torch.no_grad()
    def greedy_decode_run(self, entries: Sequence[StepEntry], num_steps: int,
                          timing: Optional[tuple] = None) -> torch.Tensor:
        """``num_steps`` greedy decode steps that stay on the device: each step's
        argmax token is the next step's input.  Every entry brings one token; the
        caller has made sure of pages for ``start + num_steps`` tokens.  Returns
        the generated tokens int32 [num_steps, S] (on the device).  ``timing`` =
        (first timed step, start event, end event) records the two CUDA events
        around the steps from the given one to the last."""
        from ..kernels import ops
        if not self.capture_graphs or any(len(e.tokens) != 1 for e in entries):
            raise StepError("greedy_decode_run needs single-token entries and capturable mixers")
        page = self.cache.page_size
        with torch.cuda.device(self.device):
            self.storage.zero_slots(self.cache.take_fresh_slots())
            last = [StepEntry(e.req, e.tokens, e.start + num_steps - 1, e.want) for e in entries]
            g = self._decode_graph(last, pad=False)            # a table wide enough for the whole run
            if g is None:
                raise StepError("too many decode graphs")
            g.fill(entries)
            S = len(entries)
            history = torch.empty((num_steps, S), dtype=torch.int32, device=self.device)
            sampled = torch.empty(S, dtype=torch.int32, device=self.device)
            for i in range(num_steps):
                if timing is not None and i == timing[0]:
                    timing[1].record()
                logits = g.run()
                ops.argmax(logits, sampled)
                ops.decode_advance(g.token_ids, g.ctx.positions, g.ctx.seq_lens, sampled, history[i])
            if timing is not None:
                timing[2].record()
            g.device_rows = None           # the rows moved on without the graph's own bookkeeping
            return history

    def poll_errors(self) -> None:
        """The same check without waiting for the GPU: looks at the error words as they were when the
        last call of this method asked for them (if that copy has arrived), raises if a kernel had
        flagged a bad index by then, and asks for a fresh copy.  An error is reported a step or two
        late; steps already queued are not held up."""
        from ..kernels import ops
        if not hasattr(self, "_err_host"):
            self._err_host = torch.zeros(2, dtype=torch.int32, pin_memory=True)
            self._err_event = None
        if self._err_event is not None:
            if not self._err_event.query():
                return
            code, gemm = int(self._err_host[0]), int(self._err_host[1])
            self._err_event = None
            if code or gemm:
                self.check_errors()            # the synchronous path words the message and clears the words
        with torch.cuda.device(self.device):
            self._err_host[0:1].copy_(self.err, non_blocking=True)
            self._err_host[1:2].copy_(ops.gemm_error_word(self.device), non_blocking=True)
            self._err_event = torch.cuda.Event()
            self._err_event.record()

    def check_errors(self) -> None:
        """Raise if a kernel of an earlier step flagged a bad index (synchronises)."""
        from ..kernels import ops
        ops.check_gemm_errors(self.device)
        code = int(self.err.item())
        if code:
            self.err.zero_()
            what = "; ".join(msg for bit, msg in _ERR_BITS.items() if code & bit)
            raise StepError(f"a kernel refused an index: {what}")
