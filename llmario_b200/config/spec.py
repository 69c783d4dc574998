"""Data that describes a model to the rest of the framework.

An architecture turns its own ``config.json`` into a :class:`ModelSpec`: a list of layers, each
made of named parts with their sizes and constants, and the order in which the layers run.  The
builder, the weight loader, the cache manager and the step function read only this data; none of
them knows which architecture produced it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A configuration is missing a key, has a wrong value, or asks for something unsupported."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` selects the implementation from the part registry of its
    role, ``params`` are that implementation's sizes and constants."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: how its parts are arranged (``block``), the token mixer, the feed-forward, and
    the prefix under which its tensors are stored."""

    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    weight_prefix: str


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.  ``layer`` indexes :attr:`ModelSpec.layers` (an index may
    occur more than once: the weights are shared, each call has a cache of its own).
    ``reads_cache_of`` is the index of an earlier entry of the run order whose cache this call
    reads instead of writing one."""

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    stored_dtype: str = "bfloat16"

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i, call in enumerate(self.run_order):
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"run order entry {i} names layer {call.layer}, "
                                  f"the model has {len(self.layers)}")
            src = call.reads_cache_of
            if src is not None:
                if not 0 <= src < i:
                    raise ConfigError(f"run order entry {i} reads the cache of entry {src}, "
                                      "which does not come before it")
                if self.run_order[src].reads_cache_of is not None:
                    raise ConfigError(f"run order entry {i} reads the cache of entry {src}, "
                                      "which has no cache of its own")
