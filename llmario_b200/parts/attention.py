"""Grouped-query attention over the paged cache, with optional per-head norm of queries and
keys and a rotary position encoding.

Order of operations as in crates/engine/model/src/forward.rs:399-485: project q, k, v; norm each
head of q and k; rotate q and k by position; store k and v in the cache; attend from the cache
(causal, optionally only the last ``window`` keys); project the result and add it to the
residual stream.  A call that reads another call's cache projects only q.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import driver, kernels
from ..cache import PagedKV
from ..config.spec import ConfigError, PartSpec
from .base import (BoundCall, StepContext, build_part, optional_tensor_of, register_part,
                   tensor_of)
from .linear import Linear


class Attention:
    graph_safe = True      # a step of single tokens reads positions and slots on the device only

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        refusal = kernels.attention_refusal(self.num_heads, self.num_kv_heads, self.head_dim)
        if refusal is not None:      # now, when the model is built, not at its first step
            raise ConfigError(f"attention: {refusal}")
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.position = (build_part("position", spec["position"], weights, dtype, device)
                         if spec.get("position") is not None else None)
        qn, kn = spec.get("q_norm"), spec.get("k_norm")
        self.q_norm = build_part("norm", qn, weights, dtype, device) if qn is not None else None
        self.k_norm = build_part("norm", kn, weights, dtype, device) if kn is not None else None
        if (self.q_norm is None) != (self.k_norm is None):
            raise ValueError("q_norm and k_norm come together")
        if self.q_norm is not None and self.q_norm.eps != self.k_norm.eps:
            raise ValueError("q_norm and k_norm must share eps")
        w = {r: tensor_of(spec, r, weights) for r in ("q", "k", "v")}
        # biases exist for the families that store them (forward.rs:399-425); tensor roles
        # "q_bias", "k_bias", "v_bias", "o_bias", each optional
        b = {r: optional_tensor_of(spec, r + "_bias", weights) for r in ("q", "k", "v", "o")}
        perm = self.position.head_permutation(self.head_dim) \
            if hasattr(self.position, "head_permutation") else None
        if perm is not None:
            # The position encoding rotates other pairs of a head than the kernels do.  A head's
            # scores do not change when queries and keys are permuted alike, so the rows of the
            # q and k projections (and what follows them per head: bias, norm gain) are permuted
            # once here and the kernels rotate their own pairs.
            perm = perm.to(device)
            for r, heads in (("q", self.num_heads), ("k", self.num_kv_heads)):
                w[r] = w[r].view(heads, self.head_dim, -1)[:, perm].reshape(w[r].shape)
                if b[r] is not None:
                    b[r] = b[r].view(heads, self.head_dim)[:, perm].reshape(-1)
            for norm in (self.q_norm, self.k_norm):
                if norm is not None:
                    norm.weight = norm.weight[perm].contiguous()
        self.qkv_proj = Linear.stacked([w["q"], w["k"], w["v"]], [b["q"], b["k"], b["v"]])
        self.q_proj = Linear(self.qkv_proj.weight[:self.q_width],      # the first rows, no copy
                             None if self.qkv_proj.bias is None else self.qkv_proj.bias[:self.q_width])
        self.o_proj = Linear(tensor_of(spec, "o", weights), b["o"])

    def cache_need(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window)

    def streamed_weights(self):
        """The matrices a step reads once: q, k, v (stacked) and the output projection."""
        return [self.qkv_proj.weight, self.o_proj.weight]

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor) -> None:
        rows = ctx.rows
        view = ctx.cache.view(call.cache_entry)
        if view is None:
            raise RuntimeError(f"run-order entry {call.index}: attention needs a cache")
        # With few rows the product is cut along K and its partial sums are added into the
        # buffer.  That buffer is created as zeros and the kernel that consumes it clears what it
        # read, which saves a clearing pass per layer.
        width = self.q_width + (2 * self.kv_width if call.writes_cache else 0)
        kept_zero = rows <= kernels.SPLIT_K_MAX_ROWS
        proj = ctx.buffer("attn.proj.%s%d" % ("z" if kept_zero else "", width), (rows, width),
                          torch.float32, zero=kept_zero)
        (self.qkv_proj if call.writes_cache else self.q_proj)(h, proj, out_is_zero=kept_zero)
        tables = self.position.rotary_tables() if self.position is not None else None
        if self.position is not None and tables is None:
            raise NotImplementedError("a position encoding that is not a rotation needs its own "
                                      "mixer")
        inv_freq, rot_dim, attn_factor = tables if tables else (None, 0, 1.0)
        angles = self.position.step_angles(ctx) if tables and hasattr(self.position, "step_angles") \
            else None
        out = ctx.buffer("attn.out", (rows, self.q_width))
        q = ctx.buffer("attn.q", (rows, self.q_width))
        if kernels.decode_fusion_ok(ctx, view, self.num_heads, self.num_kv_heads, self.head_dim,
                                    rot_dim, angles, self.window):
            # a step of single new tokens: norm, rotation, cache write and attention in one kernel
            kernels.attention_decode_fused(
                ctx, proj, out, view, call.writes_cache,
                self.q_norm.weight if self.q_norm is not None else None,
                self.k_norm.weight if self.k_norm is not None else None, angles,
                self.q_norm.eps if self.q_norm is not None else 0.0, kept_zero, self.num_heads,
                self.num_kv_heads, self.head_dim, self.scale, self.window)
            self.o_proj(out, x, accumulate=True)
            return
        kernels.qk_norm_rope_store(
            proj, q, view.k if call.writes_cache else None,
            view.v if call.writes_cache else None, view.page_stride, view.block_table,
            ctx.row_slot, ctx.row_pos,
            self.q_norm.weight if self.q_norm is not None else None,
            self.k_norm.weight if self.k_norm is not None else None,
            inv_freq, attn_factor, self.num_heads, self.num_kv_heads, self.head_dim, rot_dim,
            view.page_size, self.q_norm.eps if self.q_norm is not None else 0.0, angles,
            clear_proj=kept_zero)
        driver.attention(ctx, q, out, view, self.num_heads, self.num_kv_heads, self.head_dim,
                         self.scale, self.window)
        self.o_proj(out, x, accumulate=True)


register_part("mixer", "attention", Attention, replace=True)
