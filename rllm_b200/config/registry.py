"""One registry from an architecture's name to its model.

``config.json`` names the architecture (``architectures[0]``, else
``model_type``); the registry maps that name to a pair (typed configuration
class, function from that configuration to a ``ModelSpec``).  The generic
``DecoderModel`` is then built from the spec.  An unknown name is an error
that lists the known ones, as in the reference's ``ModelRegistry::create``
(crates/rllm-model/src/registry.rs:53-85), where an unknown name gives
``unsupported architecture``; unlike the reference's config parser, which only
warns (crates/rllm-model/src/hf_config.rs:111-116).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Tuple

from .model_config import ConfigError, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], Any]


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable[[Mapping[str, Any]], Any],
                          build_spec: Callable[[Any], Any]) -> None:
    ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def resolve_architecture(raw: Mapping[str, Any]) -> Architecture:
    _ensure_builtin()
    name = architecture_name(raw)
    if name not in ARCHITECTURES:
        raise ConfigError(f"unsupported architecture: {name!r}; known: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[name]


def load_model_description(model_dir: str) -> Tuple[Any, Any]:
    """(typed configuration, ModelSpec) of the model in ``model_dir``."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    config = arch.parse_config(raw)
    spec = arch.build_spec(config)
    spec.validate()
    return config, spec


def _ensure_builtin() -> None:
    # the built-in architecture registers itself on import
    from ..models import llama  # noqa: F401
