"""Sampling options with the reference's names, defaults and checks
(crates/rllm-core/src/request.rs:17-45 fields, :55-87 defaults, :90-119 checks).

Kept: n, presence_penalty, frequency_penalty, repetition_penalty, temperature,
top_p, top_k, min_p, seed, stop_token_ids, ignore_eos, max_tokens, min_tokens,
logit_bias, allowed_token_ids, skip_reading_prefix_cache.  Text-side options
(stop strings, detokenize, structured outputs) have no meaning for an engine
that works on token ids; ``bad_words`` is taken as token sequences
(``bad_words_token_ids``, the form the reference's sampler receives,
crates/rllm-sampling/src/sampler.rs:20): the last token of a sequence cannot
be drawn while the tokens before it are the context's last ones (the
reference masks the last token whatever the context, :95-98, so a two-token
word would ban its second token everywhere).  ``n`` > 1 asks for n samples of one prompt (the reference checks the
field, :91 and :113, and then generates one): the prompt is computed once and
the samples branch off before its last token, each with a random stream of its
own.  ``logprobs`` = N asks for the
log-probability of every generated token and of the N likeliest tokens at its place,
from the raw logits (crates/rllm-sampling/src/sampler.rs:149-160).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


class InvalidSamplingParams(ValueError):
    pass


@dataclass
class SamplingParams:
    n: int = 1
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    seed: Optional[int] = None
    stop_token_ids: Sequence[int] = ()
    ignore_eos: bool = False
    max_tokens: Optional[int] = 16
    min_tokens: int = 0
    logit_bias: Dict[int, float] = field(default_factory=dict)
    allowed_token_ids: Optional[Sequence[int]] = None
    logprobs: Optional[int] = None
    bad_words_token_ids: Sequence[Sequence[int]] = ()
    skip_reading_prefix_cache: bool = False        # compute the whole prompt even where shared pages hold a part of it

    def validate(self) -> None:
        if self.n < 1:
            raise InvalidSamplingParams("n must be >= 1")
        if self.n > 1 and self.greedy:
            raise InvalidSamplingParams("n must be 1 when sampling is greedy (temperature 0 or top_k 1)")
        if self.temperature < 0.0:
            raise InvalidSamplingParams("temperature must be >= 0")
        if not 0.0 <= self.presence_penalty <= 2.0:
            raise InvalidSamplingParams("presence_penalty must be in [0, 2]")
        if not 0.0 <= self.frequency_penalty <= 2.0:
            raise InvalidSamplingParams("frequency_penalty must be in [0, 2]")
        if self.repetition_penalty <= 0.0:
            raise InvalidSamplingParams("repetition_penalty must be > 0")
        if not 0.0 <= self.top_p <= 1.0:
            raise InvalidSamplingParams("top_p must be in [0, 1]")
        if self.min_p < 0.0 or self.min_p > 1.0:
            raise InvalidSamplingParams("min_p must be in [0, 1]")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise InvalidSamplingParams("max_tokens must be >= 1")
        if self.min_tokens < 0:
            raise InvalidSamplingParams("min_tokens must be >= 0")
        if self.logprobs is not None and not 0 <= self.logprobs <= 32:
            raise InvalidSamplingParams("logprobs must be in [0, 32]")
        if any(len(w) == 0 for w in self.bad_words_token_ids):
            raise InvalidSamplingParams("a bad word needs at least one token")

    @property
    def greedy(self) -> bool:
        """crates/rllm-sampling/src/sampler.rs:117."""
        return self.temperature <= 0.0 or self.top_k == 1

    @property
    def edits_logits(self) -> bool:
        return bool(self.logit_bias) or self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 \
            or self.presence_penalty != 0.0 or bool(self.allowed_token_ids) or self.min_tokens > 0 or bool(self.bad_words_token_ids)
