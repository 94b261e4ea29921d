"""rllm_b200: a small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

Public names are imported lazily so that host-side modules (configuration,
cache manager, scheduler) can be used without touching CUDA.
"""
__version__ = "0.1.0"

_LAZY = {
    "LLM": ("rllm_b200.llm", "LLM"),
    "SamplingParams": ("rllm_b200.sampling.params", "SamplingParams"),
    "RequestOutput": ("rllm_b200.engine.engine_core", "RequestOutput"),
    "CompletionOutput": ("rllm_b200.engine.engine_core", "CompletionOutput"),
    "Logprob": ("rllm_b200.engine.engine_core", "Logprob"),
    "EngineArgs": ("rllm_b200.config.engine_args", "EngineArgs"),
    "EngineCore": ("rllm_b200.engine.engine_core", "EngineCore"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(name)


__all__ = list(_LAZY)
