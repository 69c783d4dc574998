"""Rotary position encoding: ``freq_i = theta^(-2i/rot_dim)``, ``angle = pos * freq_scale *
freq_i``, all in 32-bit (crates/engine/cpu/src/ops.rs:46-66).  The pair that angle i turns is
(i, i + rot_dim/2) for ``rope_neox`` (``RopeKind::Neox``) and (2i, 2i + 1) for ``rope_normal``
(``RopeKind::Normal``, ops.rs:57-60).  The rotation itself is applied by the kernel that also
norms the heads and writes the cache; this part owns the constants."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..config.spec import PartSpec
from .base import register_part


class RotaryHalfSplit:
    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.rot_dim = int(spec["rot_dim"])
        self.theta = float(spec["theta"])
        self.freq_scale = float(spec.get("freq_scale", 1.0))
        self.attn_factor = float(spec.get("attn_factor", 1.0))
        if self.rot_dim % 2:
            raise ValueError("rot_dim must be even")
        i = np.arange(self.rot_dim // 2, dtype=np.float32)
        exponent = (-(np.float32(2.0) * i) / np.float32(self.rot_dim)).astype(np.float32)
        freq = np.power(np.float32(self.theta), exponent).astype(np.float32)
        freq = (np.float32(self.freq_scale) * freq).astype(np.float32)
        self.inv_freq = torch.from_numpy(freq).to(device)

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, int, float]]:
        return self.inv_freq, self.rot_dim, self.attn_factor

    def step_angles(self, ctx) -> torch.Tensor:
        """cos and sin of every row's angles, float32 [rows, rot_dim / 2, 2]: made once per
        step and shared by all layers whose rotation has the same constants."""
        key = ("rope", self.rot_dim, self.theta, self.freq_scale, self.attn_factor)
        table = ctx.shared.get(key)
        if table is None:
            from .. import kernels
            table = ctx.buffer("rope.%d.%r.%r" % (self.rot_dim, self.theta, self.freq_scale),
                               (ctx.rows, self.rot_dim // 2, 2), torch.float32)
            kernels.rope_table(ctx.row_pos, self.inv_freq, table, self.attn_factor)
            ctx.shared[key] = table
        return table


class RotaryAdjacentPairs(RotaryHalfSplit):
    """Angle i turns the pair (2i, 2i + 1).  The kernels turn (i, i + rot_dim/2); the mixer
    therefore orders each head of its query and key projections by :meth:`head_permutation`
    when it is built (scores do not depend on the order in which a head's values stand, as long
    as queries and keys stand alike), and nothing else changes."""

    def head_permutation(self, head_dim: int) -> torch.Tensor:
        """``perm`` with ``stored[j] = original[perm[j]]``: the even members of the rotated
        pairs first, then the odd ones, then what is not rotated."""
        half = self.rot_dim // 2
        perm = list(range(0, self.rot_dim, 2)) + list(range(1, self.rot_dim, 2)) \
            + list(range(self.rot_dim, head_dim))
        assert len(perm) == head_dim and perm[half] == 1
        return torch.tensor(perm, dtype=torch.long)


register_part("position", "rope_neox", RotaryHalfSplit, replace=True)
register_part("position", "rope_normal", RotaryAdjacentPairs, replace=True)
