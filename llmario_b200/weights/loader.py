"""Weights by tensor name.

The set of tensors a model needs is read off its :class:`ModelSpec`: every part lists its tensors
as ``"tensors": {role: (name, shape)}``.  A folder is checked against that set in one pass and
every fault is reported in one error: tensors that are missing, tensors nobody asked for, and
tensors of the wrong shape (the reference stops at the first ``MissingTensor`` / ``BadShape``,
crates/engine/model/src/weights.rs:91-109, 154-176).

Dtype rule.  In the bfloat16 mode 16-bit floats are kept as bfloat16, a tensor stored in 32-bit
stays 32-bit, integer tensors become int32.  In the float32 mode every float tensor is float32.
"""
from __future__ import annotations

import os
import warnings
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from ..config.spec import ModelSpec, PartSpec
from .safetensors_io import SafetensorsFolder, write_safetensors


class WeightError(ValueError):
    """The tensors of a model folder do not match what the model needs."""

    def __init__(self, missing, unexpected, wrong_shape, where: str = ""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights{' in ' + where if where else ''} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        super().__init__("\n".join(lines))


def _walk(part: PartSpec) -> Iterator[Tuple[str, Tuple[int, ...]]]:
    for key, value in part.params.items():
        if key == "tensors":
            for entry in value.values():
                name, shape = entry[0], tuple(entry[1])
                yield name, shape
        elif isinstance(value, PartSpec):
            yield from _walk(value)
        elif isinstance(value, (list, tuple)):
            for v in value:
                if isinstance(v, PartSpec):
                    yield from _walk(v)


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[int, ...]]:
    """name -> shape for every tensor the parts of ``spec`` ask for."""
    out: Dict[str, Tuple[int, ...]] = {}
    parts = [spec.embedding, spec.final_norm, spec.head]
    for layer in spec.layers:
        parts += [layer.block, layer.mixer, layer.feed_forward]
    for part in parts:
        for name, shape in _walk(part):
            if name in out and out[name] != shape:
                raise WeightError([], [], [(name, shape, out[name])], "the model's own spec")
            out[name] = shape
    return out


def optional_tensors(spec: ModelSpec) -> List[str]:
    """Tensors a folder may hold without being asked for: an output matrix stored beside a
    tied embedding is ignored (weights.rs:182-186 reads the head only when it exists)."""
    return list(spec.head.get("ignored_when_tied", ())) if spec.head.get("tied") else []


def _target_dtype(stored: torch.dtype, mode: torch.dtype) -> torch.dtype:
    if stored in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
        if mode == torch.float32:
            return torch.float32
        return torch.float32 if stored in (torch.float32, torch.float64) else torch.bfloat16
    if stored == torch.bool:
        return torch.bool
    return torch.int32


def check_tensors(spec: ModelSpec, shapes: Dict[str, Tuple[int, ...]], where: str = "") -> None:
    want = expected_tensors(spec)
    ignore = set(optional_tensors(spec))
    missing = [n for n in want if n not in shapes]
    unexpected = sorted(n for n in shapes if n not in want and n not in ignore)
    wrong = [(n, shapes[n], want[n]) for n in want if n in shapes and tuple(shapes[n]) != want[n]]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where)


def load_weights(model_dir: str, spec: ModelSpec, dtype: torch.dtype,
                 device: torch.device | str = "cpu") -> Dict[str, torch.Tensor]:
    """Read the tensors ``spec`` asks for from ``model_dir`` onto ``device``."""
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype}")
    folder = SafetensorsFolder(model_dir)
    check_tensors(spec, {n: e.shape for n, e in folder.entries.items()}, model_dir)
    ignored = [n for n in optional_tensors(spec) if n in folder.entries]
    if ignored:
        warnings.warn(f"{model_dir}: ignoring {', '.join(ignored)} (the head is tied to the "
                      "embedding)")
    out: Dict[str, torch.Tensor] = {}
    for name in expected_tensors(spec):
        t = folder.tensor(name)
        out[name] = t.to(device=device, dtype=_target_dtype(t.dtype, dtype)).contiguous()
    return out


# ------------------------------------------------------------------------------------------
# random weights
# ------------------------------------------------------------------------------------------
def random_tensors(spec: ModelSpec, seed: int, dtype: torch.dtype,
                   device: torch.device | str = "cpu", matrix_std: float = 0.02,
                   gain_std: float = 0.01) -> Dict[str, torch.Tensor]:
    """Seeded weights: matrices ~ N(0, matrix_std), one-dimensional gains 1 + N(0, gain_std).
    Every element is a function of (seed, tensor name, element index) alone
    (:mod:`.random_normal`): the values are the same bits on a CUDA device (made by the kernel
    of ``csrc/random_weights.cu``) and on the host (made by NumPy), and do not depend on the
    order of creation."""
    from .random_normal import normal_f32, tensor_key

    out: Dict[str, torch.Tensor] = {}
    device = torch.device(device)
    for name, shape in expected_tensors(spec).items():
        key = tensor_key(seed, name)
        mean, std = (1.0, gain_std) if len(shape) == 1 else (0.0, matrix_std)
        t = torch.empty(shape, dtype=dtype, device=device)
        if device.type == "cuda":
            from .. import kernels

            kernels.random_normal(t, key, mean, std)
        else:
            flat = t.view(-1)
            step = 1 << 22          # slabs bound the 64-bit temporaries
            for start in range(0, flat.numel(), step):
                n = min(step, flat.numel() - start)
                flat[start:start + n] = torch.from_numpy(normal_f32(key, start, n, mean, std)
                                                         ).to(dtype)
        out[name] = t
    return out


def write_random_model(model_dir: str, config, seed: int, dtype: Optional[torch.dtype] = None,
                       device: torch.device | str = "cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` of a model with seeded random weights.
    ``config`` is the typed configuration of a registered architecture.  ``device``: where the
    values are made before they are written (the file is the same either way)."""
    import json

    names = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}
    raw = config.to_dict()
    if dtype is None:
        dtype = names.get(raw.get("torch_dtype", "bfloat16"), torch.bfloat16)
    raw["torch_dtype"] = {v: k for k, v in names.items()}[dtype]
    os.makedirs(model_dir, exist_ok=True)
    tensors = random_tensors(config.to_spec(), seed, dtype, device)
    tensors = {n: t.cpu() for n, t in tensors.items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": str(seed)})
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    return model_dir
