"""A model put together from parts, as its :class:`ModelSpec` says.

Nothing here is specific to an architecture: the spec lists the layers, names the kind of every
part, and gives the order in which layers run (an index may occur twice; a call may read the
cache of an earlier call).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from ..config import ModelSpec, load_spec
from ..parts import BoundCall, build_part, graph_safe, part_class, streamed_weights_of
from ..weights import check_tensors, load_weights, random_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}") from None


class Model:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], dtype: torch.dtype,
                 device):
        spec.validate()
        check_tensors(spec, {n: tuple(t.shape) for n, t in weights.items()})
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.vocab_size = spec.vocab_size
        self.hidden_size = spec.hidden_size
        self.embedding = build_part("embedding", spec.embedding, weights, dtype, self.device)
        self.blocks = [part_class("block", layer.block.kind)(layer.block, layer, weights, dtype,
                                                             self.device)
                       for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, weights, dtype, self.device)
        self.head = build_part("head", spec.head, weights, dtype, self.device)
        # Cache entries.  Every block says what it keeps between steps as a list of needs; each
        # need of each run-order entry gets an entry of its own in the cache manager.  A call
        # that reads another call's cache uses that call's entries, need by need.
        self.calls: List[BoundCall] = []
        self._needs: List[Any] = []
        self._reads: List[Optional[int]] = []
        for i, call in enumerate(spec.run_order):
            block = self.blocks[call.layer]
            mine = list(block.cache_needs()) if hasattr(block, "cache_needs") \
                else [block.mixer.cache_need()]
            start = len(self._needs)
            self._needs += mine
            if call.reads_cache_of is None:
                entries = tuple(range(start, start + len(mine)))
                self._reads += [None] * len(mine)
            else:
                entries = self.calls[call.reads_cache_of].cache_entries
                if len(entries) != len(mine):
                    raise ValueError(f"run-order entry {i} reads the cache of entry "
                                     f"{call.reads_cache_of}, whose block keeps {len(entries)} "
                                     f"things where this one keeps {len(mine)}")
                self._reads += list(entries)
            self.calls.append(BoundCall(i, call.layer, call.reads_cache_of is None,
                                        entries[0] if entries else None, entries))

    def cache_needs(self) -> Tuple[List[Any], List[Optional[int]]]:
        """What every cache entry keeps between steps (PagedKV, FixedState or None), and the
        entry whose cache it reads instead of keeping one (or None)."""
        return list(self._needs), list(self._reads)

    @property
    def graph_safe(self) -> bool:
        """Whether steps of single tokens may be recorded and replayed: every part declares
        that it reads the step from device tensors only."""
        return all(graph_safe(p) for p in [self.embedding, self.final_norm, self.head]
                   + self.blocks)

    def weight_bytes(self) -> int:
        """Bytes of the matrices a decode step streams once, as the parts declare them
        (``streamed_weights()`` of every block that runs, and of the head); a matrix that
        several calls share is counted once."""
        seen, total = set(), 0
        tensors = streamed_weights_of(self.head)
        for call in self.calls:
            tensors += streamed_weights_of(self.blocks[call.layer])
        for t in tensors:
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0",
                    spec: Optional[ModelSpec] = None) -> "Model":
        """Build the model that ``config.json`` of the folder names.  ``spec`` replaces the
        layout read from the configuration (another run order, other parts) while the tensors
        still come from the folder."""
        dt = parse_dtype(dtype)
        spec = spec if spec is not None else load_spec(model_dir)
        weights = load_weights(model_dir, spec, dt, device)
        model = cls(spec, weights, dt, device)
        weights.clear()
        return model

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0",
               num_layers: Optional[int] = None) -> "Model":
        """Seeded random weights made on the device (no files).  ``config`` is a typed
        configuration of a registered architecture, or a :class:`ModelSpec`."""
        dt = parse_dtype(dtype)
        spec = config if isinstance(config, ModelSpec) else config.to_spec()
        weights = random_tensors(spec, seed, dt, device)
        model = cls(spec, weights, dt, device)
        weights.clear()
        return model
