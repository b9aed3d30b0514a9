from .base import (ConfigError, ModelConfig, build_model_spec, known_architectures, load_config,
                   lookup_architecture, parse_config, register_architecture)
from .llama import LlamaConfig

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "build_model_spec", "known_architectures",
           "load_config", "lookup_architecture", "parse_config", "register_architecture"]
