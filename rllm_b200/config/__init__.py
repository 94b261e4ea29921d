from .model_config import (ConfigError, LlamaConfig, RopeScaling, normalize_architecture,
                           normalize_dtype_name, read_config_json)
from .registry import (ARCHITECTURES, Architecture, load_model_description, register_architecture,
                       resolve_architecture)
from .engine_args import EngineArgs

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "normalize_architecture",
           "normalize_dtype_name", "read_config_json", "ARCHITECTURES", "Architecture",
           "load_model_description", "register_architecture", "resolve_architecture", "EngineArgs"]
