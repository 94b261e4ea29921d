"""What a model is made of, as data.

A model is a ``ModelSpec``: an embedding, a list of layers, the order in which
the layers run, a final norm and an output head.  A layer is a ``LayerSpec``:
an arrangement (``block``) of a mixer, a feed-forward and norms, each a
``PartSpec`` = (kind, parameters).  ``kind`` is a key of the part registries in
``rllm_b200.parts.registry``; the parameters hold every size and constant the
part needs, so a part never looks at a model configuration and does not know
which model it is in.  Layers of one model may have different kinds.

The order is data too: ``ModelSpec.order`` is a list of ``Run(layer, cache)``.
A layer index may appear twice (the same weights run twice); ``cache`` names
the cache slot that the run's mixer uses.  A run whose ``cache`` is its own
index in the order owns that slot and writes it; a run that names an earlier
run's slot reads what that run wrote and writes nothing.

The reference has one hard-wired stack instead
(crates/rllm-model/src/llama.rs:186-249).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


def _freeze(v: Any) -> Any:
    if isinstance(v, Mapping):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    if isinstance(v, (list, tuple)):
        return tuple(_freeze(x) for x in v)
    return v


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def of(kind: str, **params: Any) -> "PartSpec":
        return PartSpec(kind, _freeze(params))

    def get(self) -> Dict[str, Any]:
        return dict(self.params)

    def __getitem__(self, key: str) -> Any:
        for k, v in self.params:
            if k == key:
                return v
        raise KeyError(key)


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part takes from the weight file.

    role: "matrix": held in the run's dtype (bfloat16 or float32);
          "vector": like a matrix, but a tensor that the file stores in 32-bit
                    stays 32-bit in a bfloat16 run;
          "int":    an integer table, held as int32.
    init: how the random-weights mode draws it: ("normal", std),
          ("one_plus_normal", std), ("zeros",), ("ones",) or ("randint", high).
    An optional tensor is used when the file has it and is not drawn by the
    random-weights mode.
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple[Any, ...] = ("normal", 0.02)
    optional: bool = False           # absent from the file is not an error


@dataclass(frozen=True)
class LayerSpec:
    block: str                       # arrangement kind, e.g. "pre_norm"
    mixer: PartSpec
    ffn: PartSpec
    norms: Tuple[PartSpec, ...]      # in the order the arrangement uses them
    prefix: str                      # tensor-name prefix, e.g. "model.layers.3."


@dataclass(frozen=True)
class Run:
    layer: int
    cache: int


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[Run, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {run.layer}, the model has {len(self.layers)}")
            if not 0 <= run.cache <= i:
                raise ValueError(f"order[{i}] names cache slot {run.cache}; a run may use its own slot "
                                 f"({i}) or an earlier run's")
            if self.order[run.cache].cache != run.cache:
                raise ValueError(f"order[{i}] reads slot {run.cache}, which is not owned by run {run.cache}")


# ---------------------------------------------------------------------------
# what a mixer needs from the cache manager
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class KVPagesNeed:
    """Keys and values of every token (``window`` None) or of the last
    ``window`` tokens, in pages."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one slot of ``shape`` float32 values."""

    shape: Tuple[int, ...]
