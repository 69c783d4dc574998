"""Gated feed-forward: ``y = W_down (silu(W_gate h) * (W_up h))`` with
``silu(z) = z / (1 + exp(-z))``, no biases (crates/engine/model/src/forward.rs:500-530;
crates/engine/cpu/src/ops.rs:83-99).  Gate and up are one product over stacked rows."""
from __future__ import annotations

from typing import Dict

import torch

from .. import kernels
from ..config.spec import PartSpec
from .base import StepContext, register_part, tensor_of
from .linear import Linear


class SwiGLU:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["intermediate_size"])
        gate, up = tensor_of(spec, "gate", weights), tensor_of(spec, "up", weights)
        # For the tensor-core product gate and up rows are stored interleaved in blocks of 16
        # (16 gate rows, their 16 up rows, ...): one 128-row weight tile then holds 64 features
        # with gate and up of a feature in the same quarter of the accumulator.
        self.interleaved = kernels.gated_interleave_ok(gate, up)
        if self.interleaved:
            ff, k = gate.shape
            both = torch.stack([gate.view(ff // 16, 16, k), up.view(ff // 16, 16, k)], dim=1)
            self.gate_up = Linear(both.reshape(2 * ff, k))
        else:
            self.gate_up = Linear.stacked([gate, up])
        self.down = Linear(tensor_of(spec, "down", weights))

    def streamed_weights(self):
        return [self.gate_up.weight, self.down.weight]

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor) -> None:
        rows = ctx.rows
        act = ctx.buffer("ffn.act", (rows, self.ff))
        kernels.gate_up_silu(ctx, h, self.gate_up.weight, act, self.interleaved)
        self.down(act, x, accumulate=True)


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
