from .model_config import ConfigError, ModelConfig, Qwen3Config, read_config_json
from .registry import (Architecture, architecture_of, known_architectures, load_config,
                       register_architecture, resolve_architecture)
from .zidivik_config import ZidivikConfig
from .tidavik_config import TidavikConfig
from .toredra_config import ToredraConfig
from .engine_options import EngineOptions

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "ZidivikConfig", "TidavikConfig", "ToredraConfig", "read_config_json", "Architecture",
           "architecture_of", "known_architectures", "load_config", "register_architecture",
           "resolve_architecture", "EngineOptions"]
