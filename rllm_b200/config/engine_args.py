"""The engine's knobs, with rLLM's names, meanings and defaults.

``dtype``, ``max_model_len``, ``max_num_seqs`` (256), ``max_num_batched_tokens``
(4096), ``gpu_memory_utilization`` (0.9, within [0.01, 1]) and
``enable_prefix_caching`` are the options of ``rllm serve``
(crates/rllm-server/src/cli.rs:27-49, range check :101-107).  ``block_size``,
``num_gpu_blocks``, ``long_prefill_token_threshold`` and
``enable_chunked_prefill`` are fields of the reference's ``CacheConfig`` and
``SchedulerConfig`` (crates/rllm-core/src/config.rs:67-77, 92-101); the server
fixes the block size at 16 (crates/rllm-server/src/server.rs:34) and the
threshold at 2048 (:330).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError, normalize_dtype_name


@dataclass
class EngineArgs:
    dtype: str = "auto"
    max_model_len: Optional[int] = None
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 4096
    gpu_memory_utilization: float = 0.9
    enable_prefix_caching: bool = True
    block_size: int = 16
    num_gpu_blocks: Optional[int] = None
    long_prefill_token_threshold: int = 2048
    enable_chunked_prefill: bool = True
    enable_cuda_graphs: bool = True
    step_row_multiple: int = 128         # this engine's own: see Scheduler._trim_to_row_multiple; 0 = off
    scheduling_policy: str = "fcfs"      # or "priority" (crates/rllm-core/src/config.rs:86-98)
    seed: int = 0

    def validate(self) -> None:
        if not 0.01 <= self.gpu_memory_utilization <= 1.0:
            raise ConfigError(
                f"gpu_memory_utilization must be in range 0.01..=1.0, got {self.gpu_memory_utilization}")
        if self.max_num_seqs < 1:
            raise ConfigError("max_num_seqs must be >= 1")
        if self.max_num_batched_tokens < 1:
            raise ConfigError("max_num_batched_tokens must be >= 1")
        if self.block_size < 1:
            raise ConfigError("block_size must be >= 1")
        if self.num_gpu_blocks is not None and self.num_gpu_blocks < 1:
            raise ConfigError("num_gpu_blocks must be >= 1")
        if self.max_model_len is not None and self.max_model_len < 1:
            raise ConfigError("max_model_len must be >= 1")
        if self.long_prefill_token_threshold < 0:
            raise ConfigError("long_prefill_token_threshold must be >= 0")
        if self.step_row_multiple < 0:
            raise ConfigError("step_row_multiple must be >= 0")
        if self.scheduling_policy not in ("fcfs", "priority"):
            raise ConfigError(f"scheduling_policy must be fcfs or priority, got {self.scheduling_policy!r}")
        normalize_dtype_name(self.dtype)

    def run_dtype(self, model_dtype: str) -> str:
        """The dtype the engine computes in: ``auto`` follows config.json's
        ``torch_dtype`` (float16 checkpoints run in bfloat16: the engine has
        bfloat16 and float32 kernels only)."""
        name = normalize_dtype_name(self.dtype) or normalize_dtype_name(model_dtype) or "bfloat16"
        if name == "float16":
            if normalize_dtype_name(self.dtype) == "float16":
                raise ConfigError("dtype fp16 is not supported; use bf16 or fp32")
            name = "bfloat16"
        return name
