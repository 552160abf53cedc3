from .engine_config import EngineConfig, parse_dtype
from .model_config import ConfigError, FamupelConfig, LuporaxConfig, ModelConfig, Qwen3Config, RikanexConfig, VugudraConfig
from .registry import (build_model_spec, known_architectures, load_model_config, lookup,
                       register_model, unregister_model)

__all__ = ["EngineConfig", "parse_dtype", "ConfigError", "FamupelConfig", "LuporaxConfig", "ModelConfig", "Qwen3Config", "RikanexConfig", "VugudraConfig", "build_model_spec",
           "known_architectures", "load_model_config", "lookup", "register_model", "unregister_model"]
