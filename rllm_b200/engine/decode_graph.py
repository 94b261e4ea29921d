"""CUDA graphs for decode steps.

A step in which every request brings exactly one token launches the same
kernels with the same shapes whenever the number of requests and the width of
the block table are the same; only the contents of a few small device arrays
change.  Such a step is captured once per (number of requests, table width)
and replayed: the host then issues one copy of the packed inputs and one graph
launch instead of hundreds of kernel launches.  The kernels read lengths,
positions and page ids from device memory, never from launch arguments, so a
replay follows the step's own data.

The first two steps of a given shape run eagerly on the graph's static buffers
(their results are used, and they warm up the libraries); after the second the
same work is captured for later steps.  A capture executes nothing, so the
cache is not touched twice.

The reference captures decode for batch sizes 1..64 in powers of two on the
default stream (crates/rllm-worker/src/model_runner.rs:555-667, replay at
crates/rllm-executor/src/uniproc.rs:81-106).  Here a graph is captured on first
use, on a private stream; batches of up to 8 get a graph of their own size,
larger ones are padded to the next size of ``batch_bucket`` (steps of 4, 8, 16,
...), so that a batch that shrinks request by request keeps finding captured
graphs.  A padding row is a request of one token at position 0 whose block
table names only the storage's spare page and whose state slot is the spare
one: it reads and writes nothing that a request holds, and its logits are
dropped.
"""
from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import StepContext


def table_width_bucket(blocks: int) -> int:
    """Table widths are powers of two (at least 8) so that few graphs serve all lengths."""
    w = 8
    while w < blocks:
        w *= 2
    return w


def batch_bucket(n: int) -> int:
    """The captured batch size for n requests: n itself up to 8, then the next multiple of 4 up to 32,
    of 8 up to 64, of 16 up to 128, of 32 beyond."""
    if n <= 8:
        return n
    step = 4 if n <= 32 else (8 if n <= 64 else (16 if n <= 128 else 32))
    return -(-n // step) * step


class DecodeGraph:
    """Static buffers, context and (after the first step) the captured graph of
    decode steps with S requests and block tables of ``width`` entries."""

    def __init__(self, runner, S: int, width: int):
        self.runner, self.S, self.width = runner, S, width
        cache = runner.cache
        self.paged = list(cache.paged)
        n = 7 * S + 1 + len(self.paged) * S * width
        self.static = torch.zeros(n, dtype=torch.int32, device=runner.device)
        self.stage = torch.zeros(n, dtype=torch.int32, pin_memory=True)
        self.host = self.stage.numpy()
        self.copied = torch.cuda.Event()
        self.copied.record()
        o = [0]

        def take(k):
            v = (o[0], o[0] + k)
            o[0] += k
            return v
        self.r_tokens, self.r_pos, self.r_tseq = take(S), take(S), take(S)
        self.r_qstart, self.r_seqlens, self.r_slots, self.r_rows = take(S + 1), take(S), take(S), take(S)
        self.r_tables = [take(S * width) for _ in self.paged]
        # the parts that never change
        self.host[self.r_tseq[0]:self.r_tseq[1]] = np.arange(S)
        self.host[self.r_qstart[0]:self.r_qstart[1]] = np.arange(S + 1)
        self.host[self.r_rows[0]:self.r_rows[1]] = np.arange(S)
        sv = lambda r: self.static[r[0]:r[1]]
        tables: List[Optional[torch.Tensor]] = [None] * len(cache.needs)
        for g, r in zip(self.paged, self.r_tables):
            tables[g] = sv(r).view(S, width)
        self.token_ids = sv(self.r_tokens)
        self.rows = sv(self.r_rows)
        self.ctx = StepContext(
            num_tokens=S, num_seqs=S, num_decode=S, positions=sv(self.r_pos), token_seq=sv(self.r_tseq),
            q_start=sv(self.r_qstart), seq_lens=sv(self.r_seqlens), q_lens_host=[1] * S,
            seq_lens_host=[width * cache.page_size] * S, block_tables=tables, state_slots=sv(self.r_slots),
            state_slots_host=[], err=runner.err, act_dtype=runner.model.dtype)
        self.ctx.extras["graph"] = True
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.uses = 0
        self.live = S                  # rows that are requests; the rest pads the batch
        # what the pinned buffer holds per row: (group, admission, number of table entries written), so that an
        # unchanged block table is not written again
        self.row_state: List[Optional[tuple]] = [None] * S
        # (admission, position) of the live rows as the device buffer holds them (None: not known), as the
        # pinned buffer holds them, and whether the two differ in anything the graph reads
        self.h2d_bytes = 0             # bytes copied from the pinned buffer to the device so far
        self.device_rows: Optional[List[tuple]] = None
        self.filled_rows: List[tuple] = []
        self.dirty = True

    def fill(self, entries) -> None:
        """Pack the step's inputs into the pinned buffer and copy them over."""
        self.fill_host(entries)
        self.commit()

    def patch_tokens(self, tokens: Sequence[int]) -> None:
        """Set the input token of every request's row in the pinned buffer (after fill_host, before commit)."""
        self.host[self.r_tokens[0]:self.r_tokens[0] + len(tokens)] = tokens
        self.dirty = True

    def commit(self) -> bool:
        """Copy the pinned buffer to the device buffer the graph reads, unless that buffer already holds
        this step's inputs (``advance`` moved it there from the step before and no block table has
        changed).  Returns whether it copied: then the tokens on the device are those of the pinned buffer."""
        if not self.dirty:
            return False
        self.static.copy_(self.stage, non_blocking=True)
        self.copied.record()
        self.h2d_bytes += self.static.numel() * 4
        self.device_rows = list(self.filled_rows)
        self.dirty = False
        return True

    def advance(self, sampled: torch.Tensor, host_row: Optional[torch.Tensor]) -> None:
        """After the step's tokens were sampled: one kernel makes them the next step's input on the device
        (positions and lengths grow by one) and writes them to ``host_row`` (pinned memory) for the host.
        If the next step is these requests again and no block table changes, it needs no copy at all."""
        from ..kernels import ops
        n = sampled.numel()
        ops.decode_advance(self.token_ids, self.ctx.positions, self.ctx.seq_lens, sampled, host_row, n)
        if self.device_rows is not None and n == len(self.device_rows):
            self.device_rows = [(a, st + 1) for a, st in self.device_rows]
        else:
            self.device_rows = None

    def fill_host(self, entries) -> None:
        """Pack the step's inputs into the pinned buffer.  May run while the graph of the step before is
        still executing: that one reads the device buffer, and the copy that fed it has completed."""
        cache, S, W = self.runner.cache, self.S, self.width
        self.copied.synchronize()
        h = self.host
        self.live = len(entries)
        wrote = False                  # a block table or a padding row changed
        for s in range(len(entries), S):
            # a padding row: one token at position 0 of the spare page
            if self.row_state[s] == "pad":
                continue
            wrote = True
            self.row_state[s] = "pad"
            h[self.r_tokens[0] + s] = 0
            h[self.r_pos[0] + s] = 0
            h[self.r_seqlens[0] + s] = 1
            h[self.r_slots[0] + s] = self.runner.storage.spare_slot
            for g, r in zip(self.paged, self.r_tables):
                tab = h[r[0]:r[1]].reshape(S, W)
                tab[s, :] = -1
                tab[s, 0] = self.runner.storage.spare_page(g)
        for s, e in enumerate(entries):
            h[self.r_tokens[0] + s] = e.tokens[0]
            h[self.r_pos[0] + s] = e.start
            h[self.r_seqlens[0] + s] = e.start + 1
            h[self.r_slots[0] + s] = cache.slot(e.req)
        windowed = any(cache.needs[g].window is not None for g in self.paged)
        reqs = [e.req for e in entries]
        # a request is known by the number of its admission, not by its name: a name may come back (after
        # its request ended, or was preempted and admitted again) with other pages
        adm = [cache.requests[r] for r in reqs]
        for g, r in zip(self.paged, self.r_tables):
            # rows whose request or table length changed since they were last written (tables only grow,
            # unless a window gives pages back); the C++ side copies them into the pinned buffer
            stale = [s for s, e in enumerate(entries)
                     if windowed or self.row_state[s] != (g, adm[s], cache.table_len(e.req, g))]
            wrote = wrote or bool(stale)
            if len(stale) == len(entries):
                cache.pack_tables(reqs, g, h[r[0]:r[1]].reshape(S, W))
            else:
                tab = h[r[0]:r[1]].reshape(S, W)
                for s in stale:
                    cache.pack_tables([reqs[s]], g, tab[s:s + 1])
            if len(self.paged) == 1:
                for s in stale:
                    self.row_state[s] = (g, adm[s], cache.table_len(reqs[s], g))
            else:
                for s in stale:
                    self.row_state[s] = None      # several groups: rows are written every time
        self.filled_rows = [(adm[s], e.start) for s, e in enumerate(entries)]
        self.dirty = wrote or self.filled_rows != self.device_rows

    def run(self) -> torch.Tensor:
        """Logits float32 [live rows, vocab]; valid until the next run of this graph."""
        r = self.runner
        self.uses += 1
        if self.graph is not None:
            self.graph.replay()
            return self.logits[: self.live]
        logits = r.model.forward(self.token_ids, self.ctx, self.rows, r.storage)[: self.live]
        if self.uses >= 2 and r.capture_graphs:
            # capture the same work for the following steps (nothing executes during capture)
            # No garbage collection while capturing: freeing an older engine's graph in
            # the middle of a capture is a CUDA call that invalidates the capture.
            torch.cuda.synchronize(r.device)
            g = torch.cuda.CUDAGraph()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g, pool=r.graph_pool, capture_error_mode="thread_local"):
                    self.logits = r.model.forward(self.token_ids, self.ctx, self.rows, r.storage)
            finally:
                if gc_was_on:
                    gc.enable()
            self.graph = g
        return logits
