from .base import ConfigError, ModelConfig
from .qwen3 import FULL_ATTENTION, SLIDING_ATTENTION, Qwen3Config
from .registry import (Architecture, get_architecture, known_architectures, load_config,
                       register_architecture)

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "FULL_ATTENTION", "SLIDING_ATTENTION", "Architecture",
           "get_architecture", "known_architectures", "load_config", "register_architecture"]
