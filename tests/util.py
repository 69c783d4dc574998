"""Shared helpers of the tests: the tiny configurations, model folders with random weights,
the plain implementation's logits, and the comparison rule."""
from __future__ import annotations

import functools
import os
import random
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from plain import qwen3_plain as P

# Tiny configurations that differ in every size and option.  A and B are the two of the
# benchmark description; C adds a window on some layers, a group of three and sizes that are
# not even a multiple of four; D runs the tensor-core attention kernels.
TINY = {
    "A": dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=2048,
              use_sliding_window=False, sliding_window=None, page_size=4, seed=0),
    "B": dict(num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=3,
              head_dim=32, intermediate_size=160, vocab_size=384, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=4096,
              use_sliding_window=False, sliding_window=None, page_size=8, seed=1),
    "C": dict(num_hidden_layers=4, hidden_size=80, num_attention_heads=6, num_key_value_heads=2,
              head_dim=48, intermediate_size=112, vocab_size=301, rope_theta=500000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=1024,
              use_sliding_window=True, sliding_window=21,
              layer_types=["full_attention", "sliding_attention", "sliding_attention",
                           "full_attention"], page_size=16, seed=2),
    # D has the head size and group of the tensor-core attention kernels (tcgen05 for portions,
    # TMA-fed decode) and a window that is longer than a key tile on one layer
    "D": dict(num_hidden_layers=2, hidden_size=128, num_attention_heads=8, num_key_value_heads=2,
              head_dim=64, intermediate_size=192, vocab_size=500, rope_theta=1000000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=2048,
              use_sliding_window=True, sliding_window=150,
              layer_types=["full_attention", "sliding_attention"], page_size=16, seed=4),
    # E has sizes that no tensor-core path takes as they are: a width and a feed-forward size
    # that are no multiple of eight, five query heads on one KV head, an odd vocabulary
    "E": dict(num_hidden_layers=2, hidden_size=100, num_attention_heads=5, num_key_value_heads=1,
              head_dim=32, intermediate_size=76, vocab_size=333, rope_theta=777.0,
              rms_norm_eps=2e-5, tie_word_embeddings=False, max_position_embeddings=512,
              use_sliding_window=False, sliding_window=None, page_size=8, seed=6),
}


def config_json(name: str, dtype: str = "float32") -> dict:
    c = {k: v for k, v in TINY[name].items() if k not in ("page_size", "seed")}
    c.update(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
             attention_bias=False, rope_scaling=None, torch_dtype=dtype)
    return c


_DIRS: Dict[tuple, str] = {}
_KEEP: List[tempfile.TemporaryDirectory] = []


def model_dir(name: str, dtype: str = "float32") -> str:
    """A temporary model folder (config.json + model.safetensors) with seeded random weights,
    written by the package's own random-weights mode."""
    key = (name, dtype)
    if key not in _DIRS:
        from llmario_b200.config import Qwen3Config
        from llmario_b200.weights import write_random_model

        tmp = tempfile.TemporaryDirectory(prefix=f"llmario_tiny{name}_")
        _KEEP.append(tmp)
        cfg = Qwen3Config.from_dict(config_json(name, dtype))
        write_random_model(tmp.name, cfg, TINY[name]["seed"])
        _DIRS[key] = tmp.name
    return _DIRS[key]


@functools.lru_cache(maxsize=None)
def _plain_model(name: str, dtype: str):
    return P.load(model_dir(name, dtype), torch.float64)


def plain_logits(name: str, dtype: str, tokens: Sequence[int], kv_round: Optional[str] = None
                 ) -> np.ndarray:
    """float64 logits [T, vocab] of the plain implementation on the stored weights."""
    tensors, cfg = _plain_model(name, dtype)
    return P.forward_logits(tensors, cfg, list(tokens), kv_round=kv_round).numpy()


def random_tokens(name: str, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(TINY[name]["vocab_size"]) for _ in range(n)]


# Tolerances.  float32: the engine and the plain implementation differ by the order of 32-bit
# sums only; the reference's own bound for such differences is 1e-4 on logits of order one
# (crates/engine/model/src/forward.rs:988).  bfloat16: activations are rounded to 8 bits of
# mantissa (relative step 2^-8) at every product's input and in the cache; with a few layers
# the logits carry an error of a few steps of their own scale, bounded here by 5 % of the
# largest logit magnitude, the reference's bound for its 16-bit GPU tiles on a real model
# (crates/engine/metal/tests/backend.rs:539).
def tolerance(dtype: str, ref: np.ndarray) -> float:
    scale = max(1.0, float(np.abs(ref).max()))
    return 1e-4 * scale if dtype == "float32" else 5e-2 * float(np.abs(ref).max())


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str = "") -> None:
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got.astype(np.float64) - ref)
    tol = tolerance(dtype, ref)
    worst = np.unravel_index(np.argmax(err), err.shape)
    assert err.max() <= tol, (f"{what}: max |diff| {err.max():.3e} > {tol:.3e} at row "
                              f"{worst[0]}, column {worst[1]}")
