"""A model put together from parts, as its :class:`ModelSpec` says.

Nothing here is specific to an architecture: the spec lists the layers, names the kind of every
part, and gives the order in which layers run (an index may occur twice; a call may read the
cache of an earlier call).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from ..config import ModelSpec, load_spec
from ..parts import BoundCall, build_part, part_class
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
        self.calls: List[BoundCall] = []
        for i, call in enumerate(spec.run_order):
            owner = call.reads_cache_of if call.reads_cache_of is not None else i
            self.calls.append(BoundCall(i, call.layer, call.reads_cache_of is None, owner))

    def cache_needs(self) -> Tuple[List[Any], List[Optional[int]]]:
        """What every run-order entry keeps between steps, and whose cache it reads."""
        needs, reads = [], []
        for call, entry in zip(self.calls, self.spec.run_order):
            needs.append(self.blocks[call.layer].mixer.cache_need())
            reads.append(entry.reads_cache_of)
        return needs, reads

    def weight_bytes(self) -> int:
        """Bytes of the matrices a decode step streams once (every layer call and the head)."""
        seen, total = set(), 0

        def add(t: torch.Tensor):
            nonlocal total
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        for call in self.calls:
            b = self.blocks[call.layer]
            for part in (b.mixer, b.feed_forward):
                for v in vars(part).values():
                    if hasattr(v, "weight") and isinstance(v.weight, torch.Tensor) \
                            and v.weight.dim() == 2:
                        add(v.weight)
        add(self.head.proj.weight)
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
