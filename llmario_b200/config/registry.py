"""One registry from an architecture's name to the class that reads its configuration.

The reference picks a model family by string match on the architecture name
(crates/engine/model/src/arch.rs:204-213) and reports the list it knows
(crates/engine/bin/src/main.rs:169-179).  Here a registered class must offer
``from_dict(config_json_dict)`` and ``to_spec() -> ModelSpec``; nothing else in the package is
specific to an architecture.
"""
from __future__ import annotations

import json
import os
from typing import List, Any, Dict, Optional

from .spec import ConfigError, ModelSpec

_ARCHITECTURES: Dict[str, type] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_class: type, model_type: Optional[str] = None,
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is already registered")
    for needed in ("from_dict", "to_spec"):
        if not hasattr(config_class, needed):
            raise ConfigError(f"architecture '{name}': its class has no {needed}()")
    _ARCHITECTURES[name] = config_class
    if model_type:
        _MODEL_TYPES[model_type] = name


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: Dict[str, Any]) -> str:
    """The registered name that a ``config.json`` asks for: the first known entry of
    ``architectures``, else ``model_type``."""
    names = raw.get("architectures") or []
    for n in names:
        if n in _ARCHITECTURES:
            return n
    mt = raw.get("model_type")
    if mt in _MODEL_TYPES:
        return _MODEL_TYPES[mt]
    asked = ", ".join(map(str, names)) or str(mt)
    raise ConfigError(f"unsupported architecture: {asked}; registered: "
                      f"{', '.join(registered_architectures())}")


def config_class(name: str) -> type:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unsupported architecture: {name}; registered: "
                          f"{', '.join(registered_architectures())}")
    return _ARCHITECTURES[name]


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    with open(path) as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def _eos_ids(value) -> List[int]:
    if isinstance(value, bool):
        return []
    if isinstance(value, int):
        return [value]
    if isinstance(value, list):
        return [int(v) for v in value if isinstance(v, int) and not isinstance(v, bool)]
    return []


def load_config(model_dir: str):
    """Read ``config.json`` of a model folder into the typed configuration of its architecture.
    The end-of-sequence ids of ``generation_config.json``, when the folder has one, are merged
    with those of ``config.json`` (crates/engine/formats/src/safetensors.rs:635-651)."""
    raw = read_config_json(model_dir)
    gen_path = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen_path):
        try:
            with open(gen_path) as f:
                gen = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{gen_path}: not valid JSON ({e})") from None
        if isinstance(gen, dict):
            ids = sorted(set(_eos_ids(raw.get("eos_token_id")) + _eos_ids(gen.get("eos_token_id"))))
            if ids:
                raw = dict(raw, eos_token_id=ids)
    return config_class(resolve_architecture(raw)).from_dict(raw)


def load_spec(model_dir: str) -> ModelSpec:
    return load_config(model_dir).to_spec()
