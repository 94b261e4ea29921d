"""Log level and profiler ranges.

The reference logs through ``tracing`` with an environment filter
(src/main.rs:11-16) and a ``--log-level`` option (crates/rllm-server/src/cli.rs:79-81),
and wraps its step phases in spans: ``engine_step``
(crates/rllm-engine/src/engine_core.rs:90), ``schedule``
(crates/rllm-scheduler/src/scheduler.rs:174), ``model_forward``
(crates/rllm-executor/src/uniproc.rs:57), ``sampling``
(crates/rllm-sampling/src/sampler.rs:54).

Here: one ``logging`` logger named ``rllm_b200`` whose level comes from
``--log-level`` or the environment variable ``RLLM_LOG`` (error, warn, info,
debug, trace); at ``debug`` the engine prints one line of statistics per step.
The same four phases are NVTX ranges when ``RLLM_NVTX=1`` (off by default: a
range costs two calls a phase on the step's critical path).
"""
from __future__ import annotations

import contextlib
import logging
import os
import sys

TRACE = 5
LEVELS = {"error": logging.ERROR, "warn": logging.WARNING, "warning": logging.WARNING, "info": logging.INFO,
          "debug": logging.DEBUG, "trace": TRACE, "off": logging.CRITICAL + 1}

logger = logging.getLogger("rllm_b200")
logging.addLevelName(TRACE, "TRACE")
_configured = [False]


def set_level(name: str) -> None:
    """``name``: one of ``LEVELS``.  Installs a stderr handler on first use."""
    key = str(name).strip().lower()
    if key not in LEVELS:
        raise ValueError(f"unknown log level {name!r}; one of {sorted(LEVELS)}")
    if not _configured[0]:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter("[rllm %(levelname)s] %(message)s"))
        logger.addHandler(h)
        logger.propagate = False
        _configured[0] = True
    logger.setLevel(LEVELS[key])


if os.environ.get("RLLM_LOG"):
    set_level(os.environ["RLLM_LOG"])

NVTX = os.environ.get("RLLM_NVTX") == "1"
_null = contextlib.nullcontext()


def span(name: str):
    """A context manager: an NVTX range named ``name`` if ``RLLM_NVTX=1``, else nothing."""
    if not NVTX:
        return _null
    import torch
    return torch.cuda.nvtx.range(name)
