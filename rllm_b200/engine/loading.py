"""From a model folder to a model with weights on the device.

config.json names the architecture; the registry gives its typed configuration
and its ``ModelSpec``; the generic decoder is built from the spec and takes its
tensors by name from the folder's safetensors files, or draws them from a seed
(``random_weights``).  The reference's counterpart is
crates/rllm-model/src/runner.rs:38-67 (parse config, load all shards, build
the model by a ``match`` on the architecture).
"""
from __future__ import annotations

import json
import os
from typing import Any, Optional, Tuple

import torch

from ..config import EngineArgs, load_model_description, resolve_architecture
from ..config.model_config import ConfigError, normalize_dtype_name
from ..models.decoder import DecoderModel
from ..weights.loader import FolderSource, RandomSource, write_model_folder

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def torch_dtype_of(name: str) -> torch.dtype:
    key = normalize_dtype_name(name)
    if key not in TORCH_DTYPES:
        raise ConfigError(f"the engine computes in bfloat16 or float32, not {name!r}")
    return TORCH_DTYPES[key]


def require_cuda(device: Optional[str] = None) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("rllm_b200 needs a CUDA device (built for sm_100a); it has no CPU path")
    return torch.device(device or "cuda:0")


def load_model(model_dir: str, dtype: str = "auto", device: Optional[str] = None,
               random_weights: bool = False, seed: int = 0,
               draw_on_device: bool = False) -> Tuple[Any, DecoderModel]:
    """(typed configuration, model with weights on ``device``).  With
    ``random_weights`` the folder needs config.json only; ``draw_on_device``
    computes them with a kernel on the device (fast for large models) instead of
    on the CPU: the same values, those a written model folder would hold."""
    config, spec = load_model_description(model_dir)
    run_dtype = torch_dtype_of(EngineArgs(dtype=dtype).run_dtype(getattr(config, "torch_dtype", "bfloat16")))
    dev = require_cuda(device)
    model = DecoderModel(spec)
    if random_weights:
        source = RandomSource(model.tensor_specs(), seed, torch.float32, str(dev) if draw_on_device else "cpu")
    else:
        source = FolderSource(model_dir)
    try:
        model.load(source, run_dtype, dev)
    finally:
        source.close()
    return config, model


def write_random_model(model_dir: str, config_json: dict, seed: int, store_dtype: Optional[str] = None) -> None:
    """The random-weights mode: config.json and model.safetensors of a model
    drawn from ``seed``.  Tensors are stored in ``store_dtype`` (default: the
    configuration's ``torch_dtype``)."""
    arch = resolve_architecture(config_json)
    config = arch.parse_config(config_json)
    spec = arch.build_spec(config)
    model = DecoderModel(spec)
    name = normalize_dtype_name(store_dtype) or normalize_dtype_name(config_json.get("torch_dtype")) or "float32"
    st = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[name]
    write_model_folder(model_dir, dict(config_json), model.tensor_specs(), seed, st)
