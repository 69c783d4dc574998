"""A weight matrix ``[out][in]`` and the product ``y = x W^T`` (the reference's ``project``,
crates/engine/model/src/forward.rs:810-830).  Chooses among the hand-written matrix kernels by
dtype and size; there is no library product behind it."""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import kernels


class Linear:
    def __init__(self, weight: torch.Tensor):
        assert weight.dim() == 2
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    @classmethod
    def stacked(cls, weights: Sequence[torch.Tensor]) -> "Linear":
        """One matrix whose rows are the rows of ``weights`` in order: several projections of
        the same input become one product."""
        if len(weights) == 1:
            return cls(weights[0])
        dtypes = {w.dtype for w in weights}
        dt = torch.float32 if len(dtypes) > 1 else weights[0].dtype
        return cls(torch.cat([w.to(dt) for w in weights], dim=0))

    def __call__(self, a: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
                 out_is_zero: bool = False) -> None:
        """out (=|+=) a @ W^T.  ``out`` is float32 when accumulating.  ``out_is_zero``: the
        caller guarantees ``out`` holds zeros (saves the clearing before a split-K product)."""
        kernels.linear(a, self.weight, out, accumulate, out_is_zero)
