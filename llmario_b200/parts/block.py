"""Pre-norm residual arrangement: ``x += mixer(norm(x)); x += feed_forward(norm(x))``
(crates/engine/model/src/forward.rs:356-362).  The residual stream ``x`` is 32-bit in every
mode; the parts add into it."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import LayerSpec, PartSpec
from .base import BoundCall, StepContext, build_part, register_part


class PreNormResidualBlock:
    def __init__(self, spec: PartSpec, layer: LayerSpec, weights: Dict[str, torch.Tensor],
                 dtype, device):
        self.mixer_norm = build_part("norm", spec["mixer_norm"], weights, dtype, device)
        self.ffn_norm = build_part("norm", spec["feed_forward_norm"], weights, dtype, device)
        self.mixer = build_part("mixer", layer.mixer, weights, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, dtype,
                                       device)

    def forward(self, ctx: StepContext, call: BoundCall, x: torch.Tensor) -> None:
        h = ctx.buffer("block.h", x.shape)
        self.mixer_norm.apply(ctx, x, h)
        self.mixer.forward(ctx, call, h, x)
        self.ffn_norm.apply(ctx, x, h)
        self.feed_forward.forward(ctx, h, x)


register_part("block", "pre_norm_residual", PreNormResidualBlock, replace=True)
