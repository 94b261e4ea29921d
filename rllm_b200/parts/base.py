"""Interfaces of the parts a layer is put together from, and the per-step
context they are handed.

Every part is built from a ``PartSpec`` (its sizes and constants) and a tensor
name prefix, declares its tensors (``tensor_specs``), receives them
(``load``) and computes (``forward``).  A part never sees a model
configuration.

Interfaces
----------
Norm            forward(x_f32[T,H]) -> act[T,H]
                add_forward(x_f32[T,H] (updated in place: x += delta), delta act[T,H]) -> act[T,H]
                gather_forward(x_f32, delta|None, rows int32[R]) -> act[R,H]
PositionEncoding  apply(q[T,nq,d], k[T,nkv,d], positions) in place; optionally
                fused_rotary(device) -> (inv_freq float64[rd/2], rd) so that a mixer can
                fuse the rotation into its cache write
Mixer           cache_need() -> KVPagesNeed | StateNeed | None
                forward(x act[T,H], ctx StepContext, cache view) -> act[T,H]
FeedForward     forward(x act[T,H]) -> act[T,H]
Block           forward(h_f32[T,H], pending act[T,H]|None, ctx, cache) -> (h_f32, pending)
                where the true hidden state is h + pending (the last add is
                left to the next norm, which fuses it)

Few rows (decoding): the residual stream without norm kernels
-------------------------------------------------------------
A mixer or feed-forward that sets ``fused_residual`` takes two more forms of
its arguments.  ``residual=(h, norm)``: it adds its result into h itself (float32,
in place) and returns a ``RowSumsq``: per row, partial sums of squares of the new
h, and, if ``norm`` is given, h times that norm's weight.  And its input ``x`` may
be a ``ScaledRows`` made from such a ``RowSumsq`` by the norm (``scaled_input``):
the product that reads it multiplies each row of its result by the row's
1 / sqrt(mean(h^2) + eps), which makes it the product of the normalised h.  A
block that finds all this in its parts runs a layer as five kernels; ``pending``
between blocks is then a ``RowSumsq``, and a block that cannot use it reads h,
which is complete.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .spec import PartSpec, TensorSpec


@dataclass
class StepContext:
    """One batch of (request, its next tokens), flattened.

    Sequences with a single token this step come first (``num_decode`` of
    them).  Token i belongs to sequence ``token_seq[i]`` and has absolute
    position ``positions[i]``; sequence s owns tokens
    ``q_start[s] .. q_start[s+1]`` and holds ``seq_lens[s]`` tokens in the cache
    after this step.  ``block_tables[g]`` is the page table of cache group g,
    int32 [S, max_blocks], -1 where a page was given back.
    """

    num_tokens: int
    num_seqs: int
    num_decode: int
    positions: torch.Tensor
    token_seq: torch.Tensor
    q_start: torch.Tensor
    seq_lens: torch.Tensor
    q_lens_host: List[int]
    seq_lens_host: List[int]
    block_tables: List[torch.Tensor]
    state_slots: torch.Tensor
    state_slots_host: List[int]
    err: torch.Tensor
    act_dtype: torch.dtype = torch.bfloat16
    extras: Dict[str, object] = field(default_factory=dict)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens_host) if self.q_lens_host else 0

    @property
    def max_seq_len(self) -> int:
        return max(self.seq_lens_host) if self.seq_lens_host else 0


@dataclass
class RowSumsq:
    """h is complete.  ``parts`` float32 [P, T]: the sum over P (in the consumer's fixed
    order) is the sum of squares of row t of h.  ``scaled`` [T, H]: h times the weight
    ``scaled_by`` of the norm that is expected to read h next, rounded to the
    activation dtype; None if no such norm was named."""

    parts: torch.Tensor
    scaled: Optional[torch.Tensor] = None
    scaled_by: Optional[torch.Tensor] = None


@dataclass
class ScaledRows:
    """An RMS-normalised activation that has not been divided by its rows' root mean
    square yet: ``x`` = h * weight, ``parts`` and ``eps`` give the rows' factors
    1 / sqrt(sum(parts[:, t]) / H + eps).  Stands where an activation [T, H] stands."""

    x: torch.Tensor
    parts: torch.Tensor
    eps: float

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device


@dataclass
class KVCacheView:
    """The pages of one run's attention: K and V [pages, nkv, page_size, d]."""

    k: torch.Tensor
    v: torch.Tensor
    group: int
    writes: bool


@dataclass
class StateCacheView:
    """Fixed-size per-request state of one run: float32 [slots, *shape]."""

    state: torch.Tensor
    group: int
    writes: bool


class Part:
    # True only if ``forward``/``apply`` launches kernels without reading anything back to the host and
    # without host-to-device copies of unpinned memory: decode steps are captured in CUDA graphs only when
    # every part of every block says so.
    graph_safe = False

    def __init__(self, spec: PartSpec, prefix: str = ""):
        self.spec = spec
        self.prefix = prefix

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take this part's tensors (by full name) from ``tensors``."""

    def ignored_tensors(self) -> List[str]:
        """Full names of tensors that a weight file of this part's family may carry and the part
        does not need (buffers that it computes itself): present, they are no error."""
        return []


class Norm(Part):
    def forward(self, x: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def gather_forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                       act_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def fused_rotary(self, device=None) -> Optional[Tuple[Optional[torch.Tensor], int]]:
        """(float64 frequency table [rd/2] on ``device``, rd) if the encoding is a
        rotate-half rotation that a mixer may fuse into its cache write (rd 0:
        nothing to rotate); None if the mixer has to call ``apply``."""
        return None

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError
