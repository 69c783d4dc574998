"""Interfaces of the parts a layer is made of, and the registries that map a part's ``kind`` to
its implementation.

Roles: ``embedding``, ``mixer``, ``feed_forward``, ``norm``, ``position``, ``block``, ``head``.
A part is built from its :class:`PartSpec` (sizes, constants, tensor names), the dictionary of
loaded tensors and the compute dtype; it never looks at anything else of the model.  A new kind
is added with :func:`register_part`; nothing in the framework's files changes.

Interfaces (``ctx`` is the :class:`StepContext` of the running step):

* norm          ``apply(ctx, x_f32[rows, width], out[rows, width], rows_index=None)``
* position      ``rotary_tables()`` -> (inv_freq, rot_dim, attn_factor) for a rotation that the
                fused kernel applies, or ``None`` together with ``apply(ctx, heads_f32, n_heads)``;
                optionally ``head_permutation(head_dim)`` -> the order in which a head's values
                must stand for the kernels' pairs (i, i + rot_dim/2) to be this encoding's pairs
* mixer         ``cache_need()`` -> PagedKV | FixedState | None;
                ``forward(ctx, call, h[rows, hidden], x_f32[rows, hidden])`` adds its output to x
* feed_forward  ``forward(ctx, h[rows, hidden], x_f32[rows, hidden])`` adds its output to x
* block         ``forward(ctx, call, x_f32)``; owns the arrangement of norms, mixer, feed-forward
* embedding     ``forward(ctx, tokens_i32[rows], x_f32[rows, hidden])``
* head          ``forward(ctx, h[n, hidden], logits_f32[n, vocab])``
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..config.spec import ConfigError, PartSpec

ROLES = ("embedding", "mixer", "feed_forward", "norm", "position", "block", "head")
_REGISTRY: Dict[str, Dict[str, type]] = {r: {} for r in ROLES}


def register_part(role: str, kind: str, cls: type, replace: bool = False) -> None:
    if role not in _REGISTRY:
        raise ConfigError(f"unknown part role '{role}'; roles: {', '.join(ROLES)}")
    if kind in _REGISTRY[role] and not replace:
        raise ConfigError(f"{role} '{kind}' is already registered")
    _REGISTRY[role][kind] = cls


def unregister_part(role: str, kind: str) -> None:
    _REGISTRY[role].pop(kind, None)


def part_class(role: str, kind: str) -> type:
    try:
        return _REGISTRY[role][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(role, {}))) or "none"
        raise ConfigError(f"no {role} of kind '{kind}' is registered (known: {known})") from None


def build_part(role: str, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype: torch.dtype,
               device: torch.device):
    return part_class(role, spec.kind)(spec, weights, dtype, device)


def tensor_of(spec: PartSpec, role: str, weights: Dict[str, torch.Tensor]) -> torch.Tensor:
    """The loaded tensor that ``spec`` names for ``role``."""
    name = spec["tensors"][role][0]
    return weights[name]


def optional_tensor_of(spec: PartSpec, role: str, weights: Dict[str, torch.Tensor]
                       ) -> Optional[torch.Tensor]:
    """The loaded tensor for ``role``, or None when ``spec`` names none."""
    entry = spec["tensors"].get(role)
    return None if entry is None else weights[entry[0]]


@dataclass
class Segment:
    """The rows of one request in this step."""

    request: Any
    slot: int          # the request's row in the block tables and state tensors
    row_start: int
    rows: int
    pos_start: int     # position of the first of these rows inside the request


class Workspace:
    """Named buffers that live across steps, grown on demand, so that a step allocates nothing
    once the largest batch has been seen."""

    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[Any, torch.Tensor] = {}     # (name, dtype, shape) -> view of the buffer
        self.generation = 0     # grows whenever a buffer moves: recorded launches are stale then

    def drop(self) -> None:
        """Forget every buffer: the next step makes them anew (zero-kept ones as zeros)."""
        self._bufs.clear()
        self._views.clear()
        self.generation += 1

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype, zero: bool = False
            ) -> torch.Tensor:
        """``zero``: the buffer is created holding zeros (its users keep it that way)."""
        key = (name, dtype, tuple(shape))
        view = self._views.get(key)
        if view is not None:
            return view
        n = 1
        for d in shape:
            n *= int(d)
        buf = self._bufs.get((name, dtype))
        if buf is None or buf.numel() < n:
            make = torch.zeros if zero else torch.empty
            buf = make(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[(name, dtype)] = buf
            self.generation += 1
            # views of the buffer that was replaced are stale
            self._views = {k: v for k, v in self._views.items() if k[:2] != (name, dtype)}
        view = buf[:n].view(*shape)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[key] = view
        return view


@dataclass
class StepContext:
    """Everything a part may read about the running step."""

    rows: int
    tokens: torch.Tensor           # int32 [rows]
    row_pos: torch.Tensor          # int32 [rows]  position of each row inside its request
    row_slot: torch.Tensor         # int32 [rows]  request slot of each row
    segments: List[Segment]
    dtype: torch.dtype             # dtype of activations between parts (bfloat16 or float32)
    device: torch.device
    workspace: Workspace
    cache: Any                     # CacheManager
    fresh_slots: Sequence[int] = ()   # request slots opened since the last step
    max_pos: int = 0               # largest position in this step

    shared: Dict[Any, Any] = field(default_factory=dict)   # what parts compute once per step

    def buffer(self, name: str, shape: Sequence[int], dtype: Optional[torch.dtype] = None,
               zero: bool = False) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype or self.dtype, zero)


@dataclass
class BoundCall:
    """A run-order entry at run time: which caches (if any) it writes or reads.  A block says
    what it keeps between steps as a list of needs (``cache_needs()``); every need gets a cache
    entry of its own, numbered over the whole run order.  A block with one mixer has one."""

    index: int                     # position in the run order
    layer: int
    writes_cache: bool
    cache_entry: Optional[int]     # the (first) cache entry this call uses
    cache_entries: Tuple[int, ...] = ()   # one per need of the block, in the block's order

    def for_need(self, k: int) -> "BoundCall":
        """This call as the part that owns the block's k-th need sees it."""
        return BoundCall(self.index, self.layer, self.writes_cache, self.cache_entries[k],
                         self.cache_entries)


def streamed_weights_of(part) -> List[torch.Tensor]:
    """The matrices a part reads once per step, as the part itself declares them
    (``streamed_weights()``).  A part that declares nothing cannot be counted."""
    fn = getattr(part, "streamed_weights", None)
    if fn is None:
        raise TypeError(f"{type(part).__name__} does not declare streamed_weights(): the bytes "
                        "a step reads cannot be counted for a model with this part")
    return list(fn())


def graph_safe(part) -> bool:
    """Whether a part's work in a step of single tokens depends on the step only through
    tensors on the device (``ctx.tokens``, ``ctx.row_pos``, ``ctx.row_slot``, the caches), so
    that the step's launches can be recorded once and replayed.  A part says so with an
    attribute ``graph_safe = True``; one that does not is taken to read host data."""
    return bool(getattr(part, "graph_safe", False))
