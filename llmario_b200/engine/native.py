"""Python face of the native step driver (``csrc/step_driver.cu``).

The model is still put together from parts in Python: the registry, the run order and parts
that a user registers stay as they are.  But the blocks that are the standard arrangement of the
standard parts (pre-norm residual block, RMS norms, grouped-query attention with optional
per-head norms and half-split rotation, gated feed-forward) are described once to the native
driver, and a step runs every maximal run of such blocks with one call instead of some eight
launches per layer issued from Python.  The driver applies the same dispatch rules as
``llmario_b200.kernels`` (a test holds them to the same answers), so both ways give the same
launches; blocks it does not know run through their own ``forward``.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from ..parts.attention import Attention
from ..parts.block import PreNormResidualBlock
from ..parts.feed_forward import SwiGLU
from ..parts.norm import RmsNorm
from ..parts.position import RotaryHalfSplit


class LayerDesc(Structure):
    _fields_ = [("hidden", c_int), ("num_heads", c_int), ("num_kv_heads", c_int),
                ("head_dim", c_int), ("window", c_int), ("rot_dim", c_int),
                ("intermediate", c_int), ("interleaved", c_int),
                ("w_qkv_dtype", c_int), ("w_o_dtype", c_int), ("w_gate_up_dtype", c_int),
                ("w_down_dtype", c_int),
                ("scale", c_float), ("attn_factor", c_float), ("mixer_norm_eps", c_float),
                ("ffn_norm_eps", c_float), ("qk_norm_eps", c_float), ("pad_", c_float),
                ("mixer_norm_w", c_void_p), ("ffn_norm_w", c_void_p), ("q_norm_w", c_void_p),
                ("k_norm_w", c_void_p), ("inv_freq", c_void_p), ("w_qkv", c_void_p),
                ("w_o", c_void_p), ("w_gate_up", c_void_p), ("w_down", c_void_p)]


class CallDesc(Structure):
    _fields_ = [("layer", c_int), ("writes_cache", c_int), ("table_stride", c_int),
                ("page_size", c_int), ("n_slots", c_int), ("slot", c_int),
                ("page_stride", c_longlong), ("n_pages", c_longlong), ("k", c_void_p),
                ("v", c_void_p), ("block_table", c_void_p), ("storage", c_void_p)]


class StepDesc(Structure):
    _fields_ = [("rows", c_int), ("max_pos", c_int), ("n_segments", c_int),
                ("all_single", c_int), ("dtype", c_int), ("pad_", c_int),
                ("segments", c_void_p), ("tokens", c_void_p), ("row_pos", c_void_p),
                ("row_slot", c_void_p), ("x", c_void_p), ("status", c_void_p)]


_declared = False


def _lib():
    global _declared
    l = kernels.lib()
    if not _declared:
        l.llm_run_layers.argtypes = [POINTER(LayerDesc), POINTER(CallDesc), c_int,
                                     POINTER(StepDesc), POINTER(c_int), c_void_p]
        l.llm_run_layers.restype = c_int
        l.llm_arena_generation.argtypes = []
        l.llm_arena_generation.restype = c_longlong
        l.llm_arena_drop.argtypes = []
        l.llm_arena_drop.restype = c_int
        for name, n in (("llm_token_tile", 1), ("llm_k_splits", 3), ("llm_decode_splits", 5)):
            fn = getattr(l, name)
            fn.argtypes, fn.restype = [c_int] * n, c_int
        l.llm_set_fuse_decode.argtypes = [c_int]
        l.llm_set_fuse_decode.restype = None
        _declared = True
    return l


def arena_generation() -> int:
    """Grows whenever a buffer of the driver's arena moves: recorded steps are stale then."""
    return int(_lib().llm_arena_generation())


def arena_drop() -> None:
    """Forget the driver's buffers (after a failed step: one kept at zero may hold sums)."""
    kernels._check(_lib().llm_arena_drop(), "arena_drop")
    kernels.launches -= 1


KINDS = ("norm", "gemm_tcgen05", "gemm_simt", "rope_table", "rope_store", "decode_fused",
         "decode_tma", "decode", "flash", "merge", "tcgen05", "tcgen05_x2", "generic", "silu_mul")


def kernel_counts() -> Dict[str, int]:
    """How often the driver has launched which kind of kernel since the library was loaded."""
    l = _lib()
    l.llm_driver_counts.argtypes = [POINTER(c_longlong), c_int]
    l.llm_driver_counts.restype = c_int
    out = (c_longlong * len(KINDS))()
    n = l.llm_driver_counts(out, len(KINDS))
    assert n == len(KINDS), "the kinds of the driver and of this module differ"
    return dict(zip(KINDS, out))


def policies():
    """The native statements of the dispatch policies: (token_tile, k_splits, decode_splits)."""
    l = _lib()
    return l.llm_token_tile, l.llm_k_splits, l.llm_decode_splits


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
    if m.position is not None and type(m.position) is not RotaryHalfSplit:
        return None
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
            c = self.calls[i]
            c.layer, c.writes_cache = call.layer, int(call.writes_cache)
            c.table_stride, c.page_size = view.block_table.stride(0), view.page_size
            c.page_stride = view.page_stride
            c.k, c.v, c.block_table = view.k.data_ptr(), view.v.data_ptr(), view.block_table.data_ptr()
            st = view.storage
            if st is not None and st.is_contiguous() and st.dim() == 6:
                c.storage, c.n_pages, c.n_slots, c.slot = st.data_ptr(), st.shape[0], st.shape[1], view.slot
            else:
                c.storage, c.n_pages, c.n_slots, c.slot = None, 0, 0, 0
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
        self._step = StepDesc()
        self._launches = c_int(0)
        self._lib = _lib()
        self._status = kernels.status_words(model.device).data_ptr()
        self._segments: Optional[np.ndarray] = None

    def any(self) -> bool:
        return bool(self.runs)

    def begin_step(self, ctx, x: torch.Tensor) -> None:
        """Describe the step once; every run of layers of the step uses the description."""
        s = self._step
        s.rows, s.max_pos = ctx.rows, ctx.max_pos
        single = len(ctx.segments) == ctx.rows
        s.all_single = int(single)
        s.n_segments = len(ctx.segments)
        if single:
            s.segments = None
        else:
            seg = np.empty((len(ctx.segments), 4), dtype=np.int32)
            for i, g in enumerate(ctx.segments):
                seg[i] = (g.row_start, g.rows, g.slot, g.pos_start)
            self._segments = seg                  # kept alive for the calls of this step
            s.segments = seg.ctypes.data
        s.dtype = kernels._DT[ctx.dtype]
        s.tokens, s.row_pos, s.row_slot = ctx.tokens.data_ptr(), ctx.row_pos.data_ptr(), \
            ctx.row_slot.data_ptr()
        s.x = x.data_ptr()
        s.status = self._status

    def run(self, first: int, count: int) -> None:
        """Run-order entries ``first .. first + count`` on the step described last."""
        calls = ctypes.cast(ctypes.byref(self.calls, first * ctypes.sizeof(CallDesc)),
                            POINTER(CallDesc))
        rc = self._lib.llm_run_layers(self.layers, calls, count, ctypes.byref(self._step),
                                      ctypes.byref(self._launches), kernels._stream())
        kernels.launches += self._launches.value
        if rc != 0:
            kernels._check(rc, f"native layers {first}..{first + count - 1}")
