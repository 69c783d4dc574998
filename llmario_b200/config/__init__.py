from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .registry import (config_class, load_config, load_spec, read_config_json,
                       register_architecture, registered_architectures, resolve_architecture)
from .qwen3 import Qwen3Config

register_architecture(Qwen3Config.architecture, Qwen3Config, Qwen3Config.model_type, replace=True)

__all__ = ["ConfigError", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "Qwen3Config",
           "config_class", "load_config", "load_spec", "read_config_json",
           "register_architecture", "registered_architectures", "resolve_architecture"]
