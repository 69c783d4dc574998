"""Pre-norm residual arrangement: ``x += mixer(norm(x)); x += feed_forward(norm(x))``
(crates/engine/model/src/forward.rs:356-362).  The residual stream ``x`` is 32-bit in every
mode; the parts add into it."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import LayerSpec, PartSpec
from .base import (BoundCall, StepContext, build_part, graph_safe, register_part,
                   streamed_weights_of)


class PreNormResidualBlock:
    def __init__(self, spec: PartSpec, layer: LayerSpec, weights: Dict[str, torch.Tensor],
                 dtype, device):
        self.mixer_norm = build_part("norm", spec["mixer_norm"], weights, dtype, device)
        self.ffn_norm = build_part("norm", spec["feed_forward_norm"], weights, dtype, device)
        self.mixer = build_part("mixer", layer.mixer, weights, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, dtype,
                                       device)

    def cache_needs(self):
        """What this block keeps between steps: one need per stateful part, in a fixed order
        (here the mixer's alone).  Each need gets a cache entry; ``call.for_need(k)`` is the
        call as the owner of the k-th need sees it."""
        return [self.mixer.cache_need()]

    def streamed_weights(self):
        return streamed_weights_of(self.mixer) + streamed_weights_of(self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(graph_safe(p) for p in (self.mixer_norm, self.ffn_norm, self.mixer,
                                           self.feed_forward))

    def forward(self, ctx: StepContext, call: BoundCall, x: torch.Tensor) -> None:
        h = ctx.buffer("block.h", x.shape)
        self.mixer_norm.apply(ctx, x, h)
        self.mixer.forward(ctx, call.for_need(0) if call.cache_entries else call, h, x)
        self.ffn_norm.apply(ctx, x, h)
        self.feed_forward.forward(ctx, h, x)


register_part("block", "pre_norm_residual", PreNormResidualBlock, replace=True)
