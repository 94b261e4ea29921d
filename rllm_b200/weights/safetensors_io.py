"""Reading and writing safetensors files, and finding a model folder's shards.

The format: 8 bytes little-endian header length N, N bytes of JSON mapping a
tensor name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets count
from the end of the header), then the raw little-endian data.

Shard discovery follows the reference's three cases
(crates/rllm-model/src/loader.rs:289-379): ``model.safetensors.index.json``
(values of ``weight_map``, without duplicates, sorted; absolute paths and
``..`` are refused; every file must exist), else ``model.safetensors``, else
numbered ``model-XXXXX-of-YYYYY.safetensors`` files.
"""
from __future__ import annotations

import json
import mmap
import os
import re
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch


class WeightsError(RuntimeError):
    """A weight file or folder that cannot be used."""


_ST_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I16": (torch.int16, np.dtype("<i2"), 2),
    "I8": (torch.int8, np.dtype("i1"), 1),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "BOOL": (torch.bool, np.dtype("u1"), 1),
}
_TORCH_TO_ST = {v[0]: k for k, v in _ST_DTYPES.items()}


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read one at a time."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightsError(f"cannot open {path}: {e}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8 or n > (100 << 20):
            raise WeightsError(f"{path}: header length {n} does not fit the file")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"{path}: header is not JSON ({e})") from None
        header.pop("__metadata__", None)
        self._data_start = 8 + n
        self._size = size
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            dt, shape = info["dtype"], tuple(int(x) for x in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
            if dt not in _ST_DTYPES:
                raise WeightsError(f"{path}: tensor {name!r} has unsupported dtype {dt}")
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if e - b != count * _ST_DTYPES[dt][2] or self._data_start + e > size or b < 0:
                raise WeightsError(f"{path}: tensor {name!r} has bad offsets [{b}, {e}) for "
                                   f"shape {list(shape)} dtype {dt}")
            self.entries[name] = (dt, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self.entries[name]
        return _ST_DTYPES[dt][0], shape

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU torch tensor in its stored dtype (a copy)."""
        dt, shape, b, e = self.entries[name]
        tdt, ndt, _ = _ST_DTYPES[dt]
        count = (e - b) // ndt.itemsize
        arr = np.frombuffer(self._mm, dtype=ndt, count=count, offset=self._data_start + b)
        t = torch.from_numpy(arr.copy())
        if tdt is torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif tdt is torch.bool:
            t = t.to(torch.bool)
        return t.reshape(shape)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    """Write CPU tensors to one safetensors file (names in sorted order)."""
    header: Dict[str, dict] = {}
    offset = 0
    blobs: List[bytes] = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise WeightsError(f"cannot store dtype {t.dtype} of tensor {name!r}")
        if t.dtype is torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        elif t.dtype is torch.bool:
            raw = t.to(torch.uint8).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)


def find_weight_files(model_dir: str) -> List[str]:
    if not os.path.isdir(model_dir):
        raise WeightsError(f"model folder {model_dir!r} does not exist")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        try:
            with open(index) as f:
                weight_map = json.load(f)["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError) as e:
            raise WeightsError(f"{index}: no usable weight_map ({e})") from None
        files = sorted(set(str(v) for v in weight_map.values()))
        out = []
        for name in files:
            if os.path.isabs(name) or ".." in name.replace("\\", "/").split("/"):
                raise WeightsError(f"{index}: shard path {name!r} leaves the model folder")
            p = os.path.join(model_dir, name)
            if not os.path.isfile(p):
                raise WeightsError(f"{index} names {name!r}, which does not exist")
            out.append(p)
        return out
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    pat = re.compile(r"^model-\d+-of-\d+\.safetensors$")
    shards = sorted(n for n in os.listdir(model_dir) if pat.match(n))
    if shards:
        return [os.path.join(model_dir, n) for n in shards]
    raise WeightsError(f"no safetensors weights in {model_dir!r} (looked for "
                       "model.safetensors.index.json, model.safetensors, model-*-of-*.safetensors)")
