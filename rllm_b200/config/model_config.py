"""Typed model configuration read from a model folder's ``config.json``.

Every size and constant of the Llama decoder comes from the keys of
``config.json``; nothing of it is written into model or kernel code.

Keys, defaults and checks follow rLLM's parser
(crates/rllm-model/src/hf_config.rs:26-73 for keys and defaults, :75-118 for
the checks, :120-126 for the spellings of the architecture name).  Three keys
that the reference parses but then drops are honoured here, because the
Llama 3.2 checkpoints need them: ``rms_norm_eps`` (the reference hard-codes
1e-6, crates/rllm-model/src/llama.rs:183), ``rope_scaling`` (left ``None`` at
crates/rllm-model/src/hf_config.rs:68; the struct is
crates/rllm-core/src/config.rs:25-31) and ``tie_word_embeddings``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine runs."""


@dataclass(frozen=True)
class RopeScaling:
    """The llama3 frequency rescaling of rotary embeddings."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_json(self) -> dict:
        return asdict(self)


_LLAMA_SPELLINGS = {
    # crates/rllm-model/src/hf_config.rs:120-126
    "llama": "LlamaForCausalLM",
    "LlamaModel": "LlamaForCausalLM",
    "LLaMAForCausalLM": "LlamaForCausalLM",
    "LlamaForCausalLM": "LlamaForCausalLM",
}


def normalize_architecture(name: str) -> str:
    return _LLAMA_SPELLINGS.get(name, name)


def architecture_name(raw: Mapping[str, Any]) -> str:
    """``architectures[0]``, else ``model_type``, else ``"unknown"``
    (crates/rllm-model/src/hf_config.rs:32-37)."""
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        name = str(archs[0])
    elif raw.get("model_type"):
        name = str(raw["model_type"])
    else:
        name = "unknown"
    return normalize_architecture(name)


_DTYPE_NAMES = {
    "float32": "float32", "fp32": "float32", "f32": "float32",
    "bfloat16": "bfloat16", "bf16": "bfloat16",
    "float16": "float16", "fp16": "float16", "f16": "float16", "half": "float16",
}


def normalize_dtype_name(name: Optional[str]) -> Optional[str]:
    if name is None:
        return None
    key = str(name).lower()
    if key == "auto":
        return None
    if key not in _DTYPE_NAMES:
        raise ConfigError(f"unknown dtype {name!r}; known: auto, bf16/bfloat16, fp32/float32, fp16/float16")
    return _DTYPE_NAMES[key]


def _as_int(raw: Mapping[str, Any], key: str, default: Optional[int]) -> int:
    v = raw.get(key, None)
    if v is None:
        if default is None:
            raise ConfigError(f"config.json lacks {key!r}")
        return int(default)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json {key!r} must be an integer, got {v!r}")
    return int(v)


def _as_float(raw: Mapping[str, Any], key: str, default: float) -> float:
    v = raw.get(key, None)
    if v is None:
        return float(default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json {key!r} must be a number, got {v!r}")
    return float(v)


def _token_ids(v: Any, key: str) -> Tuple[int, ...]:
    if v is None:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (int(v),)
    if isinstance(v, (list, tuple)) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
        return tuple(int(x) for x in v)
    raise ConfigError(f"config.json {key!r} must be an integer or a list of integers, got {v!r}")


def parse_rope_scaling(v: Any) -> Optional[RopeScaling]:
    if v is None:
        return None
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json 'rope_scaling' must be an object or null, got {v!r}")
    kind = v.get("rope_type", v.get("type"))
    if kind in (None, "default"):
        return None
    if kind != "llama3":
        raise ConfigError(f"rope_scaling type {kind!r} is not supported (only 'llama3')")
    need = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
    lack = [k for k in need if k not in v]
    if lack:
        raise ConfigError(f"rope_scaling of type llama3 lacks {lack}")
    rs = RopeScaling(
        rope_type="llama3",
        factor=float(v["factor"]),
        low_freq_factor=float(v["low_freq_factor"]),
        high_freq_factor=float(v["high_freq_factor"]),
        original_max_position_embeddings=int(v["original_max_position_embeddings"]),
    )
    if rs.factor <= 0:
        raise ConfigError("rope_scaling.factor must be > 0")
    if not rs.high_freq_factor > rs.low_freq_factor:
        raise ConfigError("rope_scaling.high_freq_factor must be greater than low_freq_factor")
    if rs.original_max_position_embeddings <= 0:
        raise ConfigError("rope_scaling.original_max_position_embeddings must be > 0")
    return rs


@dataclass(frozen=True)
class LlamaConfig:
    """All sizes and constants of a Llama dense decoder."""

    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    rms_norm_eps: float
    tie_word_embeddings: bool
    hidden_act: str
    torch_dtype: str
    bos_token_id: Optional[int]
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    # ---- reading -------------------------------------------------------
    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        arch = architecture_name(raw)
        hidden = _as_int(raw, "hidden_size", 4096)
        nq = _as_int(raw, "num_attention_heads", 32)
        if hidden <= 0:
            raise ConfigError("hidden_size must be > 0")
        if nq <= 0:
            raise ConfigError("num_attention_heads must be > 0")
        nkv = _as_int(raw, "num_key_value_heads", nq)
        if hidden % nq != 0:
            raise ConfigError(f"hidden_size ({hidden}) must be divisible by num_attention_heads ({nq})")
        head_dim = _as_int(raw, "head_dim", hidden // nq)
        inter = _as_int(raw, "intermediate_size", 4 * hidden)
        dtype = normalize_dtype_name(raw.get("torch_dtype", raw.get("dtype"))) or "float16"
        act = str(raw.get("hidden_act", "silu"))
        for key in ("attention_bias", "mlp_bias"):
            if raw.get(key, False):
                raise ConfigError(f"config.json {key}=true is not supported: rLLM's Llama has no bias terms")
        bos = raw.get("bos_token_id")
        cfg = cls(
            architecture=arch,
            vocab_size=_as_int(raw, "vocab_size", 32000),
            hidden_size=hidden,
            intermediate_size=inter,
            num_hidden_layers=_as_int(raw, "num_hidden_layers", 32),
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            max_position_embeddings=_as_int(raw, "max_position_embeddings", 4096),
            rope_theta=_as_float(raw, "rope_theta", 10000.0),
            rope_scaling=parse_rope_scaling(raw.get("rope_scaling")),
            rms_norm_eps=_as_float(raw, "rms_norm_eps", 1e-6),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            hidden_act=act,
            torch_dtype=dtype,
            bos_token_id=int(bos) if isinstance(bos, int) and not isinstance(bos, bool) else None,
            eos_token_ids=_token_ids(raw.get("eos_token_id"), "eos_token_id"),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        nq, nkv, d, h = (self.num_attention_heads, self.num_key_value_heads,
                         self.head_dim, self.hidden_size)
        if nkv <= 0 or nkv > nq:
            raise ConfigError(
                f"num_key_value_heads must be > 0 and <= num_attention_heads ({nq}), got {nkv}")
        if nq % nkv != 0:
            raise ConfigError(
                f"num_attention_heads ({nq}) must be divisible by num_key_value_heads ({nkv})")
        if d != h // nq:
            raise ConfigError(
                f"head_dim ({d}) doesn't match hidden_size / num_attention_heads ({h // nq})")
        if d % 2 != 0:
            raise ConfigError(f"head_dim ({d}) must be even for rotary embeddings")
        for key in ("vocab_size", "intermediate_size", "num_hidden_layers", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be > 0")
        if self.rms_norm_eps <= 0:
            raise ConfigError("rms_norm_eps must be > 0")
        if self.rope_theta <= 0:
            raise ConfigError("rope_theta must be > 0")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")

    # ---- writing -------------------------------------------------------
    def to_json(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_json() if self.rope_scaling else None,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                   else list(self.eos_token_ids))
        return out


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {model_dir!r}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw
