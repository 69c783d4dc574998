"""A small reader and writer for the safetensors container.

File layout: 8 bytes little-endian header length N, N bytes of JSON mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the header),
then the data.  The checks are those the reference's reader makes before trusting a file
(crates/engine/formats/src/safetensors.rs:740-857): header size bound, JSON object, known dtype,
``begin <= end <= len(data)``, byte count equal to the element count times the element size, no
two tensors overlapping; for a sharded folder, no name in two shards and an index that agrees
with the shards (safetensors.rs:284-311).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

# name -> (torch dtype, numpy carrier dtype, bytes per element)
_DTYPES = {
    "F64": (torch.float64, np.float64, 8),
    "F32": (torch.float32, np.float32, 4),
    "F16": (torch.float16, np.float16, 2),
    "BF16": (torch.bfloat16, np.uint16, 2),
    "I64": (torch.int64, np.int64, 8),
    "I32": (torch.int32, np.int32, 4),
    "I16": (torch.int16, np.int16, 2),
    "I8": (torch.int8, np.int8, 1),
    "U8": (torch.uint8, np.uint8, 1),
    "BOOL": (torch.bool, np.bool_, 1),
}
_NAME_OF = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int
    path: str
    data_start: int

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


def _parse_header(path: str) -> Tuple[Dict[str, TensorEntry], Dict[str, str]]:
    size = os.path.getsize(path)
    if size < 8:
        raise SafetensorsError(f"{path}: shorter than its 8-byte length field")
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{path}: header of {n} bytes exceeds {MAX_HEADER_BYTES}")
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header of {n} bytes runs past the end of the file")
        blob = f.read(n)
    if not blob.lstrip().startswith(b"{"):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    try:
        header = json.loads(blob)
    except (json.JSONDecodeError, UnicodeDecodeError) as e:
        raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    data_len = size - 8 - n
    meta = header.pop("__metadata__", None) or {}
    entries: Dict[str, TensorEntry] = {}
    spans: List[Tuple[int, int, str]] = []
    for name, info in header.items():
        try:
            dtype, shape = info["dtype"], tuple(int(d) for d in info["shape"])
            begin, end = (int(v) for v in info["data_offsets"])
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: tensor '{name}' has a malformed entry") from None
        if dtype not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unknown dtype '{dtype}'")
        if any(d < 0 for d in shape):
            raise SafetensorsError(f"{path}: tensor '{name}' has a negative dimension")
        if not 0 <= begin <= end <= data_len:
            raise SafetensorsError(f"{path}: tensor '{name}' spans [{begin}, {end}) outside "
                                   f"the {data_len} data bytes")
        numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if end - begin != numel * _DTYPES[dtype][2]:
            raise SafetensorsError(f"{path}: tensor '{name}' holds {end - begin} bytes, its "
                                   f"shape {list(shape)} and dtype {dtype} need "
                                   f"{numel * _DTYPES[dtype][2]}")
        entries[name] = TensorEntry(name, dtype, shape, begin, end, path, 8 + n)
        if end > begin:
            spans.append((begin, end, name))
    spans.sort()
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise SafetensorsError(f"{path}: tensors '{n0}' and '{n1}' overlap")
    return entries, meta


class SafetensorsFolder:
    """The tensors of a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` lists."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        self.entries: Dict[str, TensorEntry] = {}
        self._maps: Dict[str, np.memmap] = {}
        if os.path.isfile(single):
            self.entries, _ = _parse_header(single)
        elif os.path.isfile(index):
            with open(index) as f:
                weight_map = json.load(f).get("weight_map", {})
            for shard in sorted(set(weight_map.values())):
                path = os.path.join(model_dir, shard)
                if not os.path.isfile(path):
                    raise SafetensorsError(f"{index}: shard '{shard}' does not exist")
                entries, _ = _parse_header(path)
                for name, e in entries.items():
                    if name in self.entries:
                        raise SafetensorsError(f"tensor '{name}' is in two shards")
                    self.entries[name] = e
            for name, shard in weight_map.items():
                e = self.entries.get(name)
                if e is None or os.path.basename(e.path) != shard:
                    raise SafetensorsError(f"{index}: says '{name}' is in '{shard}', "
                                           "the shards disagree")
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor "
                                   "model.safetensors.index.json")

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor backed by a private copy-on-write mapping of the file."""
        e = self.entries[name]
        mm = self._maps.get(e.path)
        if mm is None:
            mm = np.memmap(e.path, dtype=np.uint8, mode="c")
            self._maps[e.path] = mm
        tdtype, ndtype, _ = _DTYPES[e.dtype]
        raw = mm[e.data_start + e.begin: e.data_start + e.end]
        if raw.size == 0:
            return torch.empty(e.shape, dtype=tdtype)
        if (e.data_start + e.begin) % np.dtype(ndtype).itemsize:
            raw = np.array(raw)  # misaligned in the file: take an aligned copy
        arr = raw.view(ndtype)
        t = torch.from_numpy(arr)
        if e.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(e.shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor],
                      metadata: Optional[Dict[str, str]] = None) -> None:
    """Write CPU tensors in name order with an 8-byte aligned header."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAME_OF:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAME_OF[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            elif t.dtype == torch.bool:
                t = t.view(torch.uint8)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)
