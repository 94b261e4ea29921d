"""Host-side parts of the engine in C++ (no Python, no CUDA in them), built with
the system's C++ compiler on first use and loaded with ctypes, like the kernels.

``cache_core``: the pool of cache pages and the cache manager (block tables,
state slots, prefix sharing, windows), which the reference has in Rust
(crates/rllm-cache/src/block_pool.rs, manager.rs, prefix.rs).  The classes in
``rllm_b200.cache`` are thin faces of it.
"""
from .build import load_library

__all__ = ["load_library"]
