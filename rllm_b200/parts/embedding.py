"""Token embedding and output head.

Embedding: a row gather without scaling (crates/rllm-model/src/llama.rs:329-337)
that writes the float32 residual stream.  Head: logits = x . W_out^T without
bias (llama.rs:57-59, 70), W_out = ``lm_head.weight`` if the file has it, else
the embedding table (llama.rs:174-180); the logits are float32, straight from
the accumulator.  The head runs on the rows that were asked for only.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Part
from .linear import linear
from .spec import PartSpec, TensorSpec


class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, name."""

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.name = str(spec["name"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab, self.hidden))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def forward(self, token_ids: torch.Tensor, err: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        ops.embedding(token_ids, self.weight, out, err)
        return out


class OutputHead(Part):
    """params: vocab_size, hidden_size, name, tied_to (name of the embedding
    table that stands in when the file lacks ``name``; None: ``name`` is required)."""

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.name = str(spec["name"])
        self.tied_to = spec.get().get("tied_to")
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab, self.hidden), optional=self.tied_to is not None)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name] if self.name in tensors else tensors[self.tied_to]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, out_dtype=torch.float32)
