"""Typed configurations and the registry of architectures."""
from .base import (Architecture, ConfigError, ModelConfig, architectures, config_from_dict, get_architecture,
                   load_config, register_architecture)
from .gpt2 import GELU_FORMS, GPT2Config

__all__ = ["Architecture", "ConfigError", "GELU_FORMS", "GPT2Config", "ModelConfig", "architectures",
           "config_from_dict", "get_architecture", "load_config", "register_architecture"]
