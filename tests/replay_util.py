"""Helpers of the replay tests: build traces in the ways a scheduler may cut
requests, run them through trace replay, and collect the logits per request
and position."""
from __future__ import annotations

import io
import json
import os
import random
import subprocess
import sys
import tempfile
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def round64(n: int) -> int:
    return -(-n // 64) * 64


class TraceBuilder:
    """Collects steps and remembers which (request, position) each written row is."""

    def __init__(self, want=None):
        # want(request, position) -> bool: which rows' logits are asked for (default: all)
        self.want = want or (lambda rid, pos: True)
        self.steps: List[dict] = []
        self.rows: List[List[Tuple[str, int]]] = []     # per step: (request, position) of each row
        self.fed: Dict[str, int] = {}
        self.peak = 0

    def step(self, entries: Sequence[Tuple[str, Sequence[int]]], end: Sequence[str] = (),
             fork: Sequence[Tuple[str, str]] = ()):
        recs, rows = [], []
        for src, dst in fork:
            self.fed[dst] = self.fed[src]
        for rid, toks in entries:
            start = self.fed.get(rid, 0)
            wanted = [i for i in range(len(toks)) if self.want(rid, start + i)]
            recs.append({"id": rid, "tokens": list(toks), "want": wanted})
            rows += [(rid, start + i) for i in wanted]
            self.fed[rid] = start + len(toks)
        self.peak = max(self.peak, sum(round64(n) for n in self.fed.values()))
        self.steps.append({"step": len(self.steps), "entries": recs, "end": list(end)})
        if fork:
            self.steps[-1]["fork"] = [{"from": a, "to": b} for a, b in fork]
        self.rows.append(rows)
        for rid in end:
            self.fed.pop(rid, None)


def run_trace(model_dir: str, dtype: str, tb: TraceBuilder, vocab: int, page_size: int = 16,
              max_tokens: int = None, subprocess_mode: bool = False) -> Dict[Tuple[str, int], np.ndarray]:
    """(request, position) -> logits row."""
    out_dir = tempfile.mkdtemp(prefix="trace_out_")
    text = "".join(json.dumps(s) + "\n" for s in tb.steps)
    argv = ["--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens",
            str(max_tokens if max_tokens is not None else tb.peak), "--block-size", str(page_size)]
    if subprocess_mode:
        proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run")] + argv, input=text.encode(),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=600)
        assert proc.returncode == 0, proc.stderr.decode()[-4000:]
        done = proc.stdout.decode().split("\n")
    else:
        from rllm_b200.engine import replay
        old_in, old_out = sys.stdin, sys.stdout
        sys.stdin, sys.stdout = io.StringIO(text), io.StringIO()
        try:
            code = replay.main(argv)
            done = sys.stdout.getvalue().split("\n")
        finally:
            sys.stdin, sys.stdout = old_in, old_out
        assert code == 0
    assert [l for l in done if l] == [f"done {i}" for i in range(len(tb.steps))]
    got: Dict[Tuple[str, int], np.ndarray] = {}
    for i, rows in enumerate(tb.rows):
        path = os.path.join(out_dir, f"{i}.f32")
        if not rows:
            assert not os.path.exists(path)
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(len(rows), vocab)
        for r, key in enumerate(rows):
            assert key not in got, f"row {key} written twice"
            got[key] = arr[r]
    return got


def run_trace_on_model(model, tb: TraceBuilder, page_size: int = 16, max_tokens: int = None,
                       max_live: int = 8) -> Dict[Tuple[str, int], np.ndarray]:
    """The same replay on a model that is already loaded (random weights drawn on the device, say):
    ``TraceSession`` is what ``bin/trace_run`` runs for every line."""
    from rllm_b200.engine.replay import TraceSession
    session = TraceSession(model, max_tokens if max_tokens is not None else tb.peak, page_size, max_live)
    got: Dict[Tuple[str, int], np.ndarray] = {}
    for rec, rows in zip(tb.steps, tb.rows):
        arr = session.step(rec).cpu().numpy()
        assert arr.shape[0] == len(rows)
        for r, key in enumerate(rows):
            assert key not in got, f"row {key} written twice"
            got[key] = arr[r]
    session.cache.check()
    assert session.cache.usage()["num_requests"] == 0
    return got


# ---------------------------------------------------------------------------
# the ways of cutting
# ---------------------------------------------------------------------------
def trace_whole(reqs: Dict[str, List[int]], want=None) -> TraceBuilder:
    tb = TraceBuilder(want)
    for rid, toks in reqs.items():
        tb.step([(rid, toks)], end=[rid])
    return tb


def trace_tail_decode(reqs: Dict[str, List[int]], tail: int = 32, want=None) -> TraceBuilder:
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    tb = TraceBuilder(want)
    for rid, toks in reqs.items():
        head = max(0, len(toks) - tail)
        if head:
            tb.step([(rid, toks[:head])])
        for i in range(head, len(toks)):
            tb.step([(rid, toks[i:i + 1])], end=[rid] if i == len(toks) - 1 else [])
    return tb


def trace_portions(reqs: Dict[str, List[int]], seed: int = 0, want=None) -> TraceBuilder:
    """Portions of changing size, down to two tokens."""
    rng = random.Random(seed)
    tb = TraceBuilder(want)
    sizes = [7, 2, 13, 2, 5, 16, 3, 2, 33, 8, 17, 2]
    for rid, toks in reqs.items():
        pos, k = 0, rng.randrange(len(sizes))
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            tb.step([(rid, toks[pos:pos + n])], end=[rid] if pos + n == len(toks) else [])
            pos += n
    return tb


def trace_mixed(reqs: Dict[str, List[int]], seed: int = 0, live: int = 4, tail: int = 32,
                want=None) -> TraceBuilder:
    """Up to ``live`` requests at a time; each feeds portions of changing size
    (2..23 tokens), its last ``tail`` tokens one by one, and sometimes sits a
    step out; a finished request is ended and the next one starts, so its pages
    are used again."""
    rng = random.Random(seed)
    tb = TraceBuilder(want)
    waiting = list(reqs.items())
    active: List[List] = []        # [rid, tokens, pos]
    while waiting or active:
        while waiting and len(active) < live:
            rid, toks = waiting.pop(0)
            active.append([rid, toks, 0])
        entries, end = [], []
        for item in active:
            rid, toks, pos = item
            if len(active) > 1 and rng.random() < 0.15:
                continue                                   # left out of this step
            left = len(toks) - pos
            n = 1 if left <= tail else min(rng.randint(2, 23), left - tail)
            entries.append((rid, toks[pos:pos + n]))
            item[2] = pos + n
            if item[2] == len(toks):
                end.append(rid)
        if not entries:
            continue
        tb.step(entries, end=end)
        active = [it for it in active if it[2] < len(it[1])]
    return tb
