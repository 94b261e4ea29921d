"""Compiles the CUDA sources for sm_100a with nvcc and loads them with ctypes.

Every ``csrc/<name>.cu`` becomes its own shared library
``_build/<name>.<hash>.so`` next to the sources (or under the system's
temporary folder if the package folder cannot be written).  A library is
compiled the first time one of its kernels is asked for, so a program compiles
what its model and dtype need and nothing else; the hash covers the source,
the shared header and the flags, so an edited source is rebuilt and a stale
library is never loaded.  The sources include no PyTorch headers: entry points
are ``extern "C"`` and take raw pointers and a stream, which keeps a compile
at seconds.  While nvcc runs, a line is printed to stderr every few seconds.

The reference builds its kernels with nvcc per file too
(crates/rllm-kernels/build.rs:49-94) for sm_70..sm_90 (:135-153); this build
is for sm_100a only.
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
import time
from typing import Dict, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]

SOURCES = ["elementwise", "attention_simt", "attention_mma", "attention_tcgen05", "gemm_f32", "gemm_small_m", "gemm_tcgen05", "sampling", "weights_rng"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("RLLM_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (set CUDA_HOME or RLLM_NVCC); the engine has no fallback "
                           "without its CUDA kernels")


_build_dir_cache: Optional[str] = None
_dir_lock = threading.Lock()


def _build_dir() -> str:
    global _build_dir_cache
    with _dir_lock:
        if _build_dir_cache is None:
            _build_dir_cache = _pick_build_dir()
        return _build_dir_cache


def _pick_build_dir() -> str:
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"rllm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _source_hash(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for fn in sorted(os.listdir(CSRC)):
        if fn.endswith((".cuh", ".h")) or fn == name + ".cu":
            with open(os.path.join(CSRC, fn), "rb") as f:
                h.update(fn.encode())
                h.update(f.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"{name}.{_source_hash(name)}.so")


def compile_library(name: str, verbose: bool = True) -> str:
    """Compile ``csrc/<name>.cu`` if its library is missing; return the path."""
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no kernel source {src}")
    out = library_path(name)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, src]
    if verbose:
        print(f"[rllm_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env,
                            cwd=os.path.dirname(out))
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                print(f"[rllm_b200] still compiling {name}.cu ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        log = proc.communicate()[0].decode(errors="replace")
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {name}.cu:\n{log}")
    os.replace(tmp, out)
    # drop libraries of older versions of this source
    for fn in os.listdir(os.path.dirname(out)):
        if fn.startswith(name + ".") and fn.endswith(".so") and os.path.join(os.path.dirname(out), fn) != out:
            try:
                os.remove(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    if verbose:
        print(f"[rllm_b200] compiled {name}.cu in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(compile_library(name))
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True, names: Optional[List[str]] = None) -> List[str]:
    """Compile every library (in parallel); used by the build check."""
    from concurrent.futures import ThreadPoolExecutor
    names = list(names or SOURCES)
    with ThreadPoolExecutor(max_workers=min(8, len(names))) as ex:
        return list(ex.map(lambda n: compile_library(n, verbose), names))
