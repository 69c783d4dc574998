"""llmario_b200: a single-GPU inference engine for the Qwen3 dense decoder on NVIDIA B200."""
from .config import (ConfigError, ModelSpec, PartSpec, LayerSpec, LayerCall, Qwen3Config,
                     load_config, load_spec, register_architecture, registered_architectures)

__version__ = "0.1.0"
from .sampling import SamplingParams


def __getattr__(name):
    # the engine imports torch.cuda machinery; load it on first use
    if name in ("Engine", "Model", "ModelRunner", "StepEntry"):
        from . import engine as _e
        from .engine.engine import Engine
        return {"Engine": Engine, "Model": _e.Model, "ModelRunner": _e.ModelRunner,
                "StepEntry": _e.StepEntry}[name]
    raise AttributeError(name)
