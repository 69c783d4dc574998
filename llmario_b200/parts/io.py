"""Token embedding (row gather, no scaling: crates/engine/model/src/forward.rs:343-349) and the
output head (``logits = H h`` with ``H`` the output matrix or, when tied, the embedding table:
forward.rs:303-316)."""
from __future__ import annotations

from typing import Dict

import torch

from .. import kernels
from ..config.spec import PartSpec
from .base import StepContext, register_part, tensor_of
from .linear import Linear


class TokenEmbedding:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.table = tensor_of(spec, "table", weights)
        self.vocab, self.hidden = self.table.shape
        # word 1 of the library's status words: read by the host with every step's tokens
        self.err = kernels.status_words(device)[1:2] if torch.device(device).type == "cuda" \
            else torch.zeros(1, dtype=torch.int32, device=device)

    def forward(self, ctx: StepContext, tokens: torch.Tensor, x: torch.Tensor) -> None:
        kernels.embed(tokens, self.table, x, self.err)


class LinearHead:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.proj = Linear(tensor_of(spec, "weight", weights))
        self.vocab = self.proj.out_features

    def streamed_weights(self):
        return [self.proj.weight]

    def forward(self, ctx: StepContext, h: torch.Tensor, logits: torch.Tensor) -> None:
        self.proj(h, logits)


register_part("embedding", "token_embedding", TokenEmbedding, replace=True)
register_part("head", "linear_head", LinearHead, replace=True)
