"""A weight matrix ``[out][in]``, an optional bias ``[out]``, and the product ``y = x W^T + b``
(the reference's ``project``, crates/engine/model/src/forward.rs:810-830, which adds the bias
after the product when the layer has one: forward.rs:399-425).  Chooses among the hand-written
matrix kernels by dtype and size; there is no library product behind it."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        assert weight.dim() == 2
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        # a bias is kept in 32-bit whatever it was stored as: it is added in 32-bit
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        if self.bias is not None and self.bias.shape != (self.out_features,):
            raise ValueError(f"a bias of {list(self.bias.shape)} for {self.out_features} outputs")

    @classmethod
    def stacked(cls, weights: Sequence[torch.Tensor],
                biases: Optional[Sequence[Optional[torch.Tensor]]] = None) -> "Linear":
        """One matrix whose rows are the rows of ``weights`` in order: several projections of
        the same input become one product.  ``biases``: one per matrix or None for a matrix
        without (its outputs get zeros when another matrix has one)."""
        bias = None
        if biases is not None and any(b is not None for b in biases):
            bias = torch.cat([b.to(torch.float32) if b is not None else
                              torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
                              for w, b in zip(weights, biases)])
        if len(weights) == 1:
            return cls(weights[0], bias)
        dtypes = {w.dtype for w in weights}
        dt = torch.float32 if len(dtypes) > 1 else weights[0].dtype
        return cls(torch.cat([w.to(dt) for w in weights], dim=0), bias)

    def __call__(self, a: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
                 out_is_zero: bool = False) -> None:
        """out (=|+=) a @ W^T.  ``out`` is float32 when accumulating.  ``out_is_zero``: the
        caller guarantees ``out`` holds zeros (saves the clearing before a split-K product)."""
        kernels.linear(a, self.weight, out, accumulate, out_is_zero)
        if self.bias is not None:
            kernels.add_bias(out, self.bias)
