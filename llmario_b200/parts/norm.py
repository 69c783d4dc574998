"""RMS norm: ``y = x * 1/sqrt(mean(x^2) + eps) * w`` with sums and scale in 32-bit; the weight is
the plain gain (crates/engine/cpu/src/ops.rs:18-29)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.spec import PartSpec
from .base import StepContext, register_part, tensor_of


class RmsNorm:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])
        self.weight = tensor_of(spec, "weight", weights).to(device=device, dtype=torch.float32)
        assert self.weight.numel() == self.width

    def apply(self, ctx: Optional[StepContext], x: torch.Tensor, out: torch.Tensor,
              rows_index: Optional[torch.Tensor] = None) -> None:
        kernels.rms_norm(x, self.weight, out, self.eps, rows_index)


register_part("norm", "rms_norm", RmsNorm, replace=True)
