"""Python face of the native step driver (``csrc/step_driver.cu``): the C structures it is told
(mirrored field by field from ``csrc/step_driver.h``), its entry points, and the attention call
that mixers driven from Python share with it.

The driver states, in C++, which kernel serves a product or an attention call, into how many
parts K or the keys are cut, and which rows form an attention work item.  ``engine/native.py``
describes whole standard blocks to it; a mixer that is driven from Python (a part registered by a
user, or the standard attention part when the driver is switched off) calls :func:`attention`
here, so that there is one statement of the attention dispatch.
"""
from __future__ import annotations

import ctypes
import itertools
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional

import numpy as np
import torch

from . import kernels


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
                ("step_id", c_longlong), ("segments", c_void_p), ("tokens", c_void_p), ("row_pos", c_void_p),
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
        l.llm_attention_step.argtypes = [POINTER(LayerDesc), POINTER(CallDesc), POINTER(StepDesc),
                                         c_void_p, c_void_p, POINTER(c_int), c_void_p]
        l.llm_attention_step.restype = c_int
        l.llm_set_gather.argtypes = [c_int]
        l.llm_set_gather.restype = None
        _declared = True
    return l


def arena_generation() -> int:
    """Grows whenever a buffer of the driver's arena moves: recorded steps are stale then."""
    return int(_lib().llm_arena_generation())


def arena_drop() -> None:
    """Forget the driver's buffers (after a failed step: one kept at zero may hold sums)."""
    rc = _lib().llm_arena_drop()
    if rc != 0:
        raise kernels.KernelError(f"arena_drop: CUDA error {rc}")


KINDS = ("norm", "gemm_tcgen05", "gemm_simt", "rope_table", "rope_store", "decode_fused",
         "decode_tma", "decode", "flash", "merge", "tcgen05", "tcgen05_x2", "generic", "silu_mul",
         "kv_gather", "decode_persistent")


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


def arena_fill(byte: int = 0xFF) -> None:
    """Fill the driver's temporary buffers (not those it keeps at zero) with ``byte``; with 0xff
    every value in them is a NaN.  For tests: a kernel that reads what no kernel of the same
    step wrote then shows in the result."""
    l = _lib()
    l.llm_arena_fill.argtypes = [c_int]
    l.llm_arena_fill.restype = c_int
    rc = l.llm_arena_fill(int(byte))
    if rc != 0:
        raise kernels.KernelError(f"arena_fill: CUDA error {rc}")


def use_persistent_decode(on: bool) -> None:
    """Whether steps of single tokens whose decode-attention CTAs would make one to five waves
    run the persistent kernel, or one CTA per (request, KV head, part) (the default: inside a
    whole step the persistent form gains a percent at best and loses much when its CTAs do not
    all find room at once).  For measurements."""
    l = _lib()
    l.llm_set_persistent_decode.argtypes = [c_int]
    l.llm_set_persistent_decode.restype = None
    l.llm_set_persistent_decode(int(on))


def use_gather(on: bool) -> None:
    """Whether long prompt portions over a cache with small pages read gathered copies of their
    requests' keys and values (the default) or the cache as it is.  For measurements."""
    _lib().llm_set_gather(int(on))


_step_ids = itertools.count(1)


def fill_call(c: CallDesc, layer: int, writes_cache: bool, view) -> None:
    """Describe where a run-order entry's keys and values live."""
    c.layer, c.writes_cache = layer, int(writes_cache)
    c.table_stride, c.page_size = view.block_table.stride(0), view.page_size
    c.page_stride = view.page_stride
    c.k, c.v, c.block_table = view.k.data_ptr(), view.v.data_ptr(), view.block_table.data_ptr()
    st = getattr(view, "storage", None)
    if st is not None and st.is_contiguous() and st.dim() == 6:
        c.storage, c.n_pages, c.n_slots, c.slot = st.data_ptr(), st.shape[0], st.shape[1], view.slot
    else:
        c.storage, c.n_pages, c.n_slots, c.slot = None, 0, 0, 0


def describe_step(ctx, x: Optional[torch.Tensor] = None) -> StepDesc:
    """The step of ``ctx`` for the driver, made once per step (kept in ``ctx.shared``)."""
    s = ctx.shared.get("driver.step")
    if s is None:
        s = StepDesc()
        s.rows, s.max_pos = ctx.rows, ctx.max_pos
        single = all(g.rows == 1 for g in ctx.segments)
        s.all_single = int(single)
        s.n_segments = len(ctx.segments)
        if single:
            s.segments = None
        else:
            seg = np.empty((len(ctx.segments), 4), dtype=np.int32)
            for i, g in enumerate(ctx.segments):
                seg[i] = (g.row_start, g.rows, g.slot, g.pos_start)
            ctx.shared["driver.segments"] = seg          # kept alive for the calls of this step
            s.segments = seg.ctypes.data
        s.dtype = kernels._DT[ctx.dtype]
        s.step_id = next(_step_ids)
        s.tokens = ctx.tokens.data_ptr() if getattr(ctx, "tokens", None) is not None else None
        s.row_pos, s.row_slot = ctx.row_pos.data_ptr(), ctx.row_slot.data_ptr()
        s.status = kernels.status_words(ctx.row_pos.device).data_ptr()
        ctx.shared["driver.step"] = s
    if x is not None:
        s.x = x.data_ptr()
    return s


_launches = c_int(0)


def attention(ctx, q: torch.Tensor, out: torch.Tensor, view, num_heads: int, num_kv_heads: int,
              head_dim: int, scale: float, window: Optional[int]) -> None:
    """Causal attention of every row of the step over its own request's cached keys, by the
    kernels the driver chooses: bfloat16 with a head size the tensor-core kernels have goes to
    the decode kernels (single tokens and very short portions, keys split across CTAs and
    merged) and to the tcgen05 kernels (longer portions; over a cache with small pages long
    portions read a gathered copy of their keys); everything else (32-bit, other head sizes,
    very large groups) to the generic kernel."""
    kernels._cuda(q, out, view.k, view.v, view.block_table)
    assert q.dtype == out.dtype and q.is_contiguous() and out.is_contiguous()
    layer = LayerDesc()
    layer.num_heads, layer.num_kv_heads, layer.head_dim = num_heads, num_kv_heads, head_dim
    layer.scale, layer.window = scale, int(window or 0)
    call = CallDesc()
    fill_call(call, 0, True, view)
    rc = _lib().llm_attention_step(ctypes.byref(layer), ctypes.byref(call),
                                   ctypes.byref(describe_step(ctx)), q.data_ptr(), out.data_ptr(),
                                   ctypes.byref(_launches), kernels._stream())
    kernels.launches += _launches.value
    if rc != 0:
        kernels._check(rc, f"attention (head_dim {head_dim})")
