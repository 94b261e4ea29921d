"""Trace replay: feed given token ids through a model step by step and write
the logits.  Nothing is sampled.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

It drives the framework's own model, step function, cache manager and kernels
- the ones generation uses - and has no forward pass, cache or loader of its
own.  Steps come from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are asked for; all entries of a step are one batch.  ``end``: requests
that are finished after this step; their pages and slot are given back.  For a
step that asks for logits, ``<out>/<step>.f32`` holds them as little-endian
float32 [wanted, vocab] in the order of the entries and of ``want``.  After
every step a line ``done <step>`` is printed and flushed.  ``--max-tokens`` is
the most tokens live requests hold at any time (each request rounded up to a
multiple of 64); the page pool is made for exactly that many, so pages of
finished requests are used again.  An optional key ``"fork": [{"from": "a", "to": "b"}]`` makes request ``b``, before the
step's entries run, a copy of everything ``a`` has been fed so far (shared full
pages, a copied last page and state slot); both go on independently.
``--max-live`` (8) is the most requests
that are live at a time; a trace that exceeds either limit ends with exit code
3 and a message that names the step.

The reference has nothing comparable; the nearest is its hand-stepped sampler
check (crates/rllm-bench/tests/correctness.rs:120-188).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List

PAGE_SIZE = 16


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time")
    p.add_argument("--block-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    p.add_argument("--max-live", type=int, default=8,
                   help="most requests that are live at a time (state slots of the cache manager)")
    p.add_argument("--device", default="cuda:0")
    return p


class TraceError(RuntimeError):
    """A trace asks for more pages or live requests than the session was given."""


class TraceSession:
    """The state of one replay: a cache manager and storage sized for ``max_tokens``
    tokens and ``max_live`` requests around a loaded model, and the model runner that
    generation uses.  ``step`` takes one record of the trace and returns the logits
    at the wanted places (float32 [wanted, vocab] on the device)."""

    def __init__(self, model, max_tokens: int, block_size: int = PAGE_SIZE, max_live: int = 8):
        from ..cache import CacheManager, CacheStorage
        from .runner import ModelRunner
        self.model = model
        page = int(block_size)
        num_pages = max(1, -(-int(max_tokens) // page))
        paged = [n for n in model.layout.groups if hasattr(n, "num_kv_heads")]
        self.max_tokens, self.max_live = int(max_tokens), max(1, int(max_live))
        self.cache = CacheManager(model.layout.groups, page, [num_pages] * len(paged), self.max_live)
        self.storage = CacheStorage(model.layout, page, [num_pages] * len(paged), self.max_live, model.dtype,
                                    model.device)
        self.runner = ModelRunner(model, self.cache, self.storage)
        self.fed: Dict[str, int] = {}

    def step(self, rec: dict):
        import torch

        from .runner import StepEntry
        step = rec.get("step")
        for f in rec.get("fork", []):
            src, dst = str(f["from"]), str(f["to"])
            if src not in self.fed or dst in self.fed:
                raise TraceError(f"step {step}: cannot fork {src!r} into {dst!r}")
            made = self.cache.fork(src, dst, self.fed[src])
            if made is None:
                raise TraceError(f"step {step}: no page or slot left to fork {src!r}")
            with torch.cuda.device(self.model.device):
                self.storage.copy_for_fork(*made)
            self.fed[dst] = self.fed[src]
        entries = []
        for e in rec.get("entries", []):
            rid, tokens = str(e["id"]), list(e["tokens"])
            if not tokens:
                continue
            if rid not in self.fed:
                if not self.cache.has_free_slot():
                    raise TraceError(f"step {step}: request {rid!r} would be live request number "
                                     f"{len(self.fed) + 1}; --max-live is {self.max_live}")
                self.cache.admit(rid)
                self.fed[rid] = 0
            start = self.fed[rid]
            if not self.cache.ensure(rid, start, start + len(tokens)):
                raise TraceError(f"step {step}: request {rid!r} needs more pages than --max-tokens "
                                 f"{self.max_tokens} leaves free")
            entries.append(StepEntry(rid, tokens, start, list(e.get("want", []))))
            self.fed[rid] = start + len(tokens)
        logits = self.runner.step(entries)
        self.runner.check_errors()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in self.fed:
                self.cache.free(rid)
                del self.fed[rid]
        return logits


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    print("[trace_run] loading", args.model, file=sys.stderr, flush=True)
    import numpy as np
    import torch

    from .loading import load_model

    os.makedirs(args.out, exist_ok=True)
    _, model = load_model(args.model, dtype=args.dtype, device=args.device)
    session = TraceSession(model, args.max_tokens, args.block_size, args.max_live)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        try:
            logits = session.step(rec)
        except TraceError as e:
            print(f"trace_run: {e}", file=sys.stderr)
            return 3
        if logits.shape[0]:
            logits.cpu().numpy().astype("<f4").tofile(os.path.join(args.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
