"""Compiles ``native/csrc/<name>.cc`` with g++ into ``_build/<name>.<hash>.so``
next to the sources (or under the system's temporary folder if the package
folder cannot be written) the first time it is asked for, and loads it with
ctypes.  The hash covers the source and the flags, so an edited source is
rebuilt and a stale library is never loaded.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
from typing import Dict

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]
SOURCES = ["cache_core"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class NativeBuildError(RuntimeError):
    pass


def _compiler() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return cand
    raise NativeBuildError("no C++ compiler found (set CXX); the engine's cache manager is C++")


def _build_dir() -> str:
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"rllm_b200_native_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(name: str) -> str:
    h = hashlib.sha256(" ".join(CXX_FLAGS).encode())
    with open(os.path.join(CSRC, name + ".cc"), "rb") as f:
        h.update(f.read())
    return os.path.join(_build_dir(), f"{name}.{h.hexdigest()[:16]}.so")


def compile_library(name: str, verbose: bool = True) -> str:
    src = os.path.join(CSRC, name + ".cc")
    if not os.path.isfile(src):
        raise NativeBuildError(f"no source {src}")
    out = library_path(name)
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [_compiler()] + CXX_FLAGS + ["-o", tmp, src]
    if verbose:
        print(f"[rllm_b200] compiling {name}.cc ...", file=sys.stderr, flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise NativeBuildError(f"{cmd[0]} failed on {name}.cc:\n{proc.stdout}")
    os.replace(tmp, out)
    for fn in os.listdir(os.path.dirname(out)):        # libraries of older versions of this source
        if fn.startswith(name + ".") and fn.endswith(".so") and os.path.join(os.path.dirname(out), fn) != out:
            try:
                os.remove(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    return out


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = _loaded[name] = ctypes.CDLL(compile_library(name))
        return lib


def build_all(verbose: bool = True):
    return [compile_library(n, verbose) for n in SOURCES]
