from .llama import ConfigError, LlamaConfig, RopeScaling
from .registry import (architectures, config_from_dict, load_config,
                       register_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "architectures",
           "config_from_dict", "load_config", "register_architecture",
           "LayerSpec", "ModelSpec", "PartSpec", "RunEntry"]
