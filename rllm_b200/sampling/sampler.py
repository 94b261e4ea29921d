"""From logits to next tokens, on the device.

The order of the reference's pipeline is kept
(crates/rllm-sampling/src/sampler.rs:62-169): logit bias, repetition,
frequency and presence penalties, bad words, allowed-token mask, EOS
suppression below ``min_tokens`` (the three masks set logits to -inf, so their
order among themselves changes nothing); then greedy, or temperature, top-k, top-p, min-p and a draw.
The kernels are in ``kernels/csrc/sampling.cu``, which also lists the
deliberate differences (per-request Philox stream, exact fixed-point mass,
ties).  The host's part is to turn the requests' histories and options into
the flat arrays the kernels take; logits never leave the device.
"""
from __future__ import annotations

from collections import Counter
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


@dataclass
class SamplingRow:
    """One row of logits and the request it belongs to."""

    params: SamplingParams
    seed: int                       # the request's seed, resolved
    gen_index: int                  # index of the token being generated (0 for the first)
    context: Sequence[int] = ()     # prompt + generated tokens; read only if penalties are on
    eos_token_ids: Sequence[int] = ()


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def _option_buffers(self, R: int):
        """(numpy view of a pinned int32 buffer, device buffer, event of the last copy from it); pinned
        buffers are used in turn so that filling one does not wait for the copy of the call before."""
        if not hasattr(self, "_pinned") or self._pinned[0][0].numel() < 8 * R:
            n = max(8 * R, 8 * 256)
            self._pinned = [(torch.zeros(n, dtype=torch.int32, pin_memory=True), torch.cuda.Event()) for _ in range(4)]
            self._devbuf = [torch.zeros(n, dtype=torch.int32, device=self.device) for _ in range(4)]
            self._slot = 0
        self._slot = (self._slot + 1) % 4
        t, ev = self._pinned[self._slot]
        return t.numpy(), self._devbuf[self._slot], ev

    def _dev(self, arr: np.ndarray) -> torch.Tensor:
        return torch.from_numpy(arr).to(self.device, non_blocking=False)

    def apply_processors(self, logits: torch.Tensor, rows: Sequence[SamplingRow]) -> None:
        """Biases, penalties and masks, in place."""
        e_rows: List[int] = []
        e_tok: List[int] = []
        e_cnt: List[int] = []
        e_bias: List[float] = []
        sup_rows: List[int] = []
        sup_tok: List[int] = []
        allowed_start = [0]
        allowed: List[int] = []
        any_allowed = False
        R = len(rows)
        rep = np.ones(R, dtype=np.float32)
        freq = np.zeros(R, dtype=np.float32)
        pres = np.zeros(R, dtype=np.float32)
        for r, row in enumerate(rows):
            p = row.params
            penalised = p.repetition_penalty != 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0
            counts = Counter(row.context) if penalised else {}
            rep[r], freq[r], pres[r] = p.repetition_penalty, p.frequency_penalty, p.presence_penalty
            touched = set(counts) | set(p.logit_bias)
            for t in touched:
                e_rows.append(r)
                e_tok.append(int(t))
                e_cnt.append(int(counts.get(t, 0)))
                e_bias.append(float(p.logit_bias.get(t, 0.0)))
            if p.allowed_token_ids:
                allowed += sorted(set(int(t) for t in p.allowed_token_ids))
                any_allowed = True
            allowed_start.append(len(allowed))
            if p.min_tokens > 0 and row.gen_index < p.min_tokens:
                for t in row.eos_token_ids:
                    sup_rows.append(r)
                    sup_tok.append(int(t))
            for word in p.bad_words_token_ids:
                # the word's last token, where the context ends with the tokens before it
                k = len(word) - 1
                if k == 0 or (len(row.context) >= k and list(row.context[len(row.context) - k:]) == [int(t) for t in word[:k]]):
                    sup_rows.append(r)
                    sup_tok.append(int(word[-1]))
        if e_rows:
            ops.logit_edits(logits, self._dev(np.asarray(e_rows, np.int32)), self._dev(np.asarray(e_tok, np.int32)),
                            self._dev(np.asarray(e_cnt, np.int32)), self._dev(np.asarray(e_bias, np.float32)),
                            self._dev(rep), self._dev(freq), self._dev(pres))
        if any_allowed or sup_rows:
            ops.logit_mask(logits,
                           self._dev(np.asarray(allowed_start, np.int32)) if any_allowed else None,
                           self._dev(np.asarray(allowed or [0], np.int32)) if any_allowed else None,
                           self._dev(np.asarray(sup_rows, np.int32)) if sup_rows else None,
                           self._dev(np.asarray(sup_tok, np.int32)) if sup_rows else None)

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        """int32 [R]: the lowest index of the largest logit of every row."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        if logits.shape[0]:
            ops.argmax(logits, out)
        return out

    @torch.no_grad()
    def sample(self, logits: torch.Tensor, rows: Sequence[SamplingRow]) -> torch.Tensor:
        """int32 [R] next tokens on the device.  ``logits`` float32 [R, V] may be
        edited in place."""
        R = logits.shape[0]
        assert R == len(rows)
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        if R == 0:
            return out
        if any(row.params.edits_logits for row in rows):
            self.apply_processors(logits, rows)
        if all(row.params.greedy for row in rows):
            ops.argmax(logits, out)
            return out
        # all per-row options in one pinned buffer and one copy: int64 first (seeds, token indices),
        # then float32 bits (temperature, top_p, min_p) and int32 (top_k)
        host, dev, copied = self._option_buffers(R)
        copied.synchronize()                      # the copy that last read this pinned buffer is through
        s = host[: 4 * R].view(np.int64).reshape(2, R)
        f = host[4 * R: 7 * R].view(np.float32).reshape(3, R)
        k = host[7 * R: 8 * R]
        for r, row in enumerate(rows):
            p = row.params
            f[0, r], f[1, r], f[2, r] = p.temperature, p.top_p, p.min_p
            k[r] = p.top_k
            s[0, r] = np.int64(np.uint64(row.seed & 0xFFFFFFFFFFFFFFFF).astype(np.int64))
            s[1, r] = row.gen_index
        with torch.cuda.device(self.device):
            dev[: 8 * R].copy_(self._pinned[self._slot][0][: 8 * R], non_blocking=True)
            copied.record()
        sd = dev[: 4 * R].view(torch.int64).view(2, R)
        fd = dev[4 * R: 7 * R].view(torch.float32).view(3, R)
        kd = dev[7 * R: 8 * R]
        V = logits.shape[1]
        # the top-k / top-p kernels are left out when no row uses them
        select = any(1 < row.params.top_k < V or 0.0 < row.params.top_p < 1.0 for row in rows)
        ops.sample(logits, fd[0], kd, fd[1], fd[2], sd[0], sd[1], out, with_select=select)
        return out
