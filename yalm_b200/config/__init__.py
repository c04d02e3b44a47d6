from .golulix import GolulixConfig
from .llama import ConfigError, LlamaConfig, RopeScaling
from .rudazen import RudazenConfig
from .registry import (architectures, config_from_dict, load_config,
                       register_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

__all__ = ["ConfigError", "GolulixConfig", "LlamaConfig", "RudazenConfig", "RopeScaling", "architectures",
           "config_from_dict", "load_config", "register_architecture",
           "LayerSpec", "ModelSpec", "PartSpec", "RunEntry"]
