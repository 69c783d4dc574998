"""llmario_b200: a single-GPU inference engine for the Qwen3 dense decoder on NVIDIA B200."""
from .config import (ConfigError, ModelSpec, PartSpec, LayerSpec, LayerCall, Qwen3Config,
                     load_config, load_spec, register_architecture, registered_architectures)

__version__ = "0.1.0"
