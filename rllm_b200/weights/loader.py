"""Weights by tensor name: from a model folder, or drawn from a seed.

A model's parts declare the tensors they take (``TensorSpec``: name, shape,
role).  ``load_tensors`` takes exactly those from a ``WeightSource`` and checks
the whole set first: if tensors are missing, unexpected or of the wrong shape
it raises ONE ``WeightsMismatch`` that lists all of them.  The reference takes
tensors by name too (crates/rllm-model/src/llama.rs:167-256: ``remove(name)``,
error ``missing <name>``) but stops at the first missing one, checks no shape
and ignores leftovers.

Held dtypes: a "matrix" is held in the run's dtype (bfloat16 or float32); a
"vector" stored in 32-bit stays 32-bit even in a bfloat16 run; an "int" table
becomes int32.

The random source draws each tensor from a counter-based generator keyed by
the model seed and a hash of the tensor's name (``counter_rng``), so a
tensor's values do not depend on which other tensors exist, nor on where they
are drawn: the CPU and the GPU give the same bits.  The reference has only an
unseeded test helper (crates/rllm-model/src/llama.rs:367-428: N(0, 0.02)
matrices, norms of ones).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import SafetensorsFile, WeightsError, find_weight_files, write_safetensors

class WeightsMismatch(WeightsError):
    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_kind: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = ["the weights do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong dtype ({len(self.wrong_kind)}): " + ", ".join(
                f"{n} is {got}" for n, got in self.wrong_kind))
        super().__init__("\n".join(lines))


class WeightSource:
    def names(self) -> List[str]:
        raise NotImplementedError

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        raise NotImplementedError

    def read(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def close(self) -> None:
        pass


class FolderSource(WeightSource):
    """All safetensors shards of a model folder."""

    def __init__(self, model_dir: str):
        self.files = [SafetensorsFile(p) for p in find_weight_files(model_dir)]
        self.where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self.where[n] = f

    def names(self) -> List[str]:
        return list(self.where)

    def info(self, name):
        return self.where[name].info(name)

    def read(self, name):
        return self.where[name].read(name)

    def close(self):
        for f in self.files:
            f.close()


def _fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for b in text.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def tensor_key(name: str, seed: int) -> int:
    """The 64-bit key of a tensor's random stream: the model seed and a hash of the name."""
    return ((int(seed) * 0x9E3779B97F4A7C15) ^ _fnv1a64(name)) & 0xFFFFFFFFFFFFFFFF


def draw_tensor(spec: TensorSpec, seed: int, device: str = "cpu") -> torch.Tensor:
    """The random tensor for ``spec`` under ``seed``, float32 (int64 for "int").
    The values are a function of (seed, tensor name, element index) alone
    (``counter_rng``): drawn on the CPU they are what a written model folder
    holds, and a CUDA ``device`` computes the same bits with a kernel, which is
    much faster for large models."""
    kind = spec.init[0]
    n = 1
    for d in spec.shape:
        n *= int(d)
    key = tensor_key(spec.name, seed)
    on_gpu = str(device).startswith("cuda")
    if kind in ("normal", "one_plus_normal"):
        if on_gpu:
            from ..kernels import ops
            out = torch.empty(spec.shape, dtype=torch.float32, device=device)
            ops.draw_normal(out, key, float(spec.init[1]), kind == "one_plus_normal")
            return out
        from . import counter_rng
        v = counter_rng.normal(n, key, float(spec.init[1]), kind == "one_plus_normal")
        return torch.from_numpy(v).reshape(spec.shape)
    if kind == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    if kind == "ones":
        return torch.ones(spec.shape, dtype=torch.float32, device=device)
    if kind == "randint":
        if on_gpu:
            from ..kernels import ops
            out = torch.empty(spec.shape, dtype=torch.int32, device=device)
            ops.draw_randint(out, key, int(spec.init[1]))
            return out.to(torch.int64)
        from . import counter_rng
        return torch.from_numpy(counter_rng.randint(n, key, int(spec.init[1]))).reshape(spec.shape).to(torch.int64)
    raise WeightsError(f"tensor {spec.name!r}: unknown init rule {spec.init!r}")


class RandomSource(WeightSource):
    """Draws the tensors of ``specs`` from ``seed``; optional tensors are absent."""

    def __init__(self, specs: Iterable[TensorSpec], seed: int, store_dtype: torch.dtype = torch.float32,
                 device: str = "cpu"):
        self.specs = {s.name: s for s in specs if not s.optional}
        self.seed = int(seed)
        self.store_dtype = store_dtype
        self.device = device

    def names(self):
        return list(self.specs)

    def _dtype(self, s: TensorSpec) -> torch.dtype:
        return torch.int32 if s.role == "int" else self.store_dtype

    def info(self, name):
        s = self.specs[name]
        return self._dtype(s), tuple(s.shape)

    def read(self, name):
        s = self.specs[name]
        return draw_tensor(s, self.seed, self.device).to(self._dtype(s))


def _held_dtype(spec: TensorSpec, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "int":
        return torch.int32
    if spec.role == "vector" and stored in (torch.float32, torch.float64):
        return torch.float32
    return run_dtype


def check_tensors(specs: Sequence[TensorSpec], source: WeightSource, ignored: Iterable[str] = ()) -> None:
    """``ignored``: full names that the model's parts declared as present-but-unused."""
    have = set(source.names())
    want = {s.name: s for s in specs}
    skip = set(ignored)
    missing = sorted(n for n, s in want.items() if n not in have and not s.optional)
    unexpected = sorted(n for n in have if n not in want and n not in skip)
    wrong_shape, wrong_kind = [], []
    for n, s in want.items():
        if n not in have:
            continue
        dt, shape = source.info(n)
        if tuple(shape) != tuple(s.shape):
            wrong_shape.append((n, tuple(shape), tuple(s.shape)))
        if (s.role == "int") == dt.is_floating_point:
            wrong_kind.append((n, str(dt)))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightsMismatch(missing, unexpected, sorted(wrong_shape), sorted(wrong_kind))


def load_tensors(specs: Sequence[TensorSpec], source: WeightSource, run_dtype: torch.dtype,
                 device: torch.device, ignored: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """name -> tensor on ``device`` for every spec the source has."""
    check_tensors(specs, source, ignored)
    have = set(source.names())
    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        if s.name not in have:
            continue
        t = source.read(s.name)
        out[s.name] = t.to(_held_dtype(s, t.dtype, run_dtype)).to(device).contiguous()
    return out


def write_model_folder(model_dir: str, config_json: dict, specs: Sequence[TensorSpec], seed: int,
                       store_dtype: torch.dtype) -> None:
    """config.json and model.safetensors of a random model."""
    os.makedirs(model_dir, exist_ok=True)
    src = RandomSource(specs, seed, store_dtype)
    tensors = {n: src.read(n) for n in src.names()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config_json, f, indent=1)
