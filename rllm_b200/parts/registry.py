"""Registries from a part's kind to the class that builds it.

A new mixer, feed-forward, norm, position encoding or block arrangement is
added by registering a class here under a new kind; model specs then name the
kind.  Nothing else in the framework has to change: the weight loader, the
random-weights writer, the cache manager and the step function work from what
the parts declare (``tensor_specs``, ``cache_need``).

The reference's registry maps only whole architectures
(crates/rllm-model/src/registry.rs:53-85); parts are hard-wired there.
"""
from __future__ import annotations

from typing import Callable, Dict, Type

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}

_TABLES = {
    "mixer": MIXERS,
    "feed_forward": FEED_FORWARDS,
    "norm": NORMS,
    "position_encoding": POSITION_ENCODINGS,
    "block": BLOCKS,
}


def register_part(family: str, kind: str) -> Callable[[type], type]:
    """Class decorator: ``@register_part("mixer", "attention")``."""
    table = _TABLES[family]

    def deco(cls: type) -> type:
        table[kind] = cls
        return cls

    return deco


def build_part(family: str, spec, **kwargs):
    table = _TABLES[family]
    if spec.kind not in table:
        raise KeyError(f"no {family} of kind {spec.kind!r} is registered; known: {sorted(table)}")
    return table[spec.kind](spec, **kwargs)
