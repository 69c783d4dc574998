"""Roofline arithmetic shared by ``bench.py`` and the command line's ``bench``.

A decode step has to read every weight matrix it uses once and the cached keys and values of the
live requests; a prompt portion has to do the flops of its products and of its attention.  The
peaks they are held against are measured ones when a ``MEASURED_PEAKS.json`` is found (next to
the package, or where ``LLMARIO_PEAKS`` points), else a stated fallback.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks(path: Optional[str] = None) -> Dict[str, Any]:
    """hbm_gbs, bf16_tflops (burst), bf16_tflops_sustained and ``source``: "measured" or
    "fallback"."""
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    for cand in (path, os.environ.get("LLMARIO_PEAKS"), os.path.join(root, "MEASURED_PEAKS.json")):
        if cand and os.path.isfile(cand):
            try:
                with open(cand) as f:
                    raw = json.load(f)
            except (OSError, ValueError):
                continue
            out: Dict[str, Any] = dict(FALLBACK_PEAKS)
            for k in FALLBACK_PEAKS:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
            return out
    return dict(FALLBACK_PEAKS, source="fallback")


def kv_bytes_per_token(runner) -> int:
    """Bytes of keys and values one cached token takes over all layers."""
    cache = runner.cache
    return cache.storage_bytes(runner.model.dtype) // (cache.groups[0].n_pages * runner.page_size)


def decode_step_bytes(model, runner, batch: int, mean_context: float) -> float:
    """Bytes a decode step of ``batch`` requests has to read: the streamed weights once and
    ``mean_context`` cached tokens per request."""
    return model.weight_bytes() + batch * mean_context * kv_bytes_per_token(runner)


def prefill_flops(model, tokens: int, first_position: int = 0, logit_rows: int = 1) -> float:
    """Flops of one prompt portion of ``tokens`` tokens that starts at ``first_position``: two
    per weight of the layer matrices and token, causal attention (scores and weighted values
    over the keys each token sees), and the head for ``logit_rows`` rows."""
    head = sum(t.numel() for t in model.head.streamed_weights())
    layer_params = model.weight_bytes() / _element_size(model) - head
    flops = 2.0 * tokens * layer_params + 2.0 * logit_rows * head
    for call in model.calls:
        mixer = getattr(model.blocks[call.layer], "mixer", None)
        heads, hd = getattr(mixer, "num_heads", 0), getattr(mixer, "head_dim", 0)
        # sum over the portion's tokens of the keys each sees, times 2 products of 2 flops
        seen = tokens * first_position + tokens * (tokens + 1) / 2.0
        flops += 4.0 * heads * hd * seen
    return flops


def _element_size(model) -> int:
    import torch

    return torch.empty((), dtype=model.dtype).element_size()


def fraction(achieved: float, peak: float) -> float:
    return achieved / peak if peak else 0.0
