"""Whole standard blocks described to the native step driver.

The model is still put together from parts in Python: the registry, the run order and parts
that a user registers stay as they are.  But the blocks that are the standard arrangement of the
standard parts (pre-norm residual block, RMS norms, grouped-query attention with optional
per-head norms and half-split rotation, gated feed-forward) are described once to the driver
(``csrc/step_driver.cu``), and a step runs every maximal run of such blocks with one call instead
of some eight launches per layer issued from Python.  Blocks the driver does not know run through
their own ``forward``.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int
from typing import Dict, Optional, Tuple

import torch

from .. import driver, kernels
from ..driver import (CallDesc, LayerDesc, StepDesc, arena_drop, arena_generation,  # noqa: F401
                      kernel_counts, policies)
from ..parts.attention import Attention
from ..parts.block import PreNormResidualBlock
from ..parts.feed_forward import SwiGLU
from ..parts.norm import RmsNorm
from ..parts.position import RotaryAdjacentPairs, RotaryHalfSplit


def describe_block(block, shared_tables: Dict[Tuple, torch.Tensor]) -> Optional[LayerDesc]:
    """The description of ``block`` for the native driver, or None when it is not exactly the
    standard arrangement of the standard parts (a subclass or a user's part may behave
    otherwise: it keeps running through its own ``forward``)."""
    if type(block) is not PreNormResidualBlock:
        return None
    m, f = block.mixer, block.feed_forward
    if type(m) is not Attention or type(f) is not SwiGLU:
        return None
    if type(block.mixer_norm) is not RmsNorm or type(block.ffn_norm) is not RmsNorm:
        return None
    if m.position is not None and type(m.position) not in (RotaryHalfSplit, RotaryAdjacentPairs):
        return None         # (adjacent pairs: the mixer has ordered its rows for the kernels' pairs)
    if any(lin.bias is not None for lin in (m.qkv_proj, m.o_proj, f.gate_up, f.down)):
        return None         # a bias is a launch of its own behind the product: the part's forward
    if m.q_norm is not None and (type(m.q_norm) is not RmsNorm or type(m.k_norm) is not RmsNorm):
        return None
    d = LayerDesc()
    d.hidden = m.hidden
    d.num_heads, d.num_kv_heads, d.head_dim = m.num_heads, m.num_kv_heads, m.head_dim
    d.window = int(m.window or 0)
    d.intermediate = f.ff
    d.interleaved = int(f.interleaved)
    d.scale = m.scale
    d.mixer_norm_eps, d.ffn_norm_eps = block.mixer_norm.eps, block.ffn_norm.eps
    d.mixer_norm_w, d.ffn_norm_w = block.mixer_norm.weight.data_ptr(), block.ffn_norm.weight.data_ptr()
    if m.q_norm is not None:
        d.qk_norm_eps = m.q_norm.eps
        d.q_norm_w, d.k_norm_w = m.q_norm.weight.data_ptr(), m.k_norm.weight.data_ptr()
    if m.position is not None:
        p = m.position
        # layers whose rotation has the same constants share one table of angles per step: the
        # driver tells tables apart by the address of the frequencies
        key = (p.rot_dim, p.theta, p.freq_scale, p.attn_factor, p.inv_freq.device)
        table = shared_tables.setdefault(key, p.inv_freq)
        d.rot_dim, d.attn_factor, d.inv_freq = p.rot_dim, p.attn_factor, table.data_ptr()
    else:
        d.rot_dim, d.attn_factor = 0, 1.0
    for name, lin in (("w_qkv", m.qkv_proj), ("w_o", m.o_proj), ("w_gate_up", f.gate_up),
                      ("w_down", f.down)):
        w = lin.weight
        if not w.is_contiguous() or w.dtype not in kernels._DT:
            return None
        setattr(d, name, w.data_ptr())
        setattr(d, name + "_dtype", kernels._DT[w.dtype])
    return d


class NativeLayers:
    """The native descriptions of a model's blocks and run-order entries, and the call that
    runs a stretch of the run order."""

    def __init__(self, model, cache):
        self._keep: Dict[Tuple, torch.Tensor] = {}
        descs = [describe_block(b, self._keep) for b in model.blocks]
        self.native_layer = [d is not None for d in descs]
        self.n_layers = len(descs)
        self.layers = (LayerDesc * max(1, self.n_layers))(*[d if d is not None else LayerDesc()
                                                            for d in descs])
        n = len(model.calls)
        self.calls = (CallDesc * max(1, n))()
        self.native_call = []
        for i, call in enumerate(model.calls):
            ok = self.native_layer[call.layer]
            view = cache.view(call.cache_entry) if ok and call.cache_entry is not None else None
            if view is None:
                self.native_call.append(False)
                continue
            driver.fill_call(self.calls[i], call.layer, call.writes_cache, view)
            self.native_call.append(True)
        # maximal runs of native calls: [(first, count)], and which run starts at a given call
        self.runs: Dict[int, int] = {}
        i = 0
        while i < n:
            if self.native_call[i]:
                j = i
                while j < n and self.native_call[j]:
                    j += 1
                self.runs[i] = j - i
                i = j
            else:
                i += 1
        self._step: Optional[StepDesc] = None
        self._launches = c_int(0)
        self._lib = driver._lib()

    def any(self) -> bool:
        return bool(self.runs)

    def begin_step(self, ctx, x: torch.Tensor) -> None:
        """Describe the step once; every run of layers of the step uses the description."""
        self._step = driver.describe_step(ctx, x)

    def run(self, first: int, count: int) -> None:
        """Run-order entries ``first .. first + count`` on the step described last."""
        calls = ctypes.cast(ctypes.byref(self.calls, first * ctypes.sizeof(CallDesc)),
                            POINTER(CallDesc))
        rc = self._lib.llm_run_layers(self.layers, calls, count, ctypes.byref(self._step),
                                      ctypes.byref(self._launches), kernels._stream())
        kernels.launches += self._launches.value
        if rc != 0:
            kernels._check(rc, f"native layers {first}..{first + count - 1}")
