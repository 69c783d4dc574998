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
    # W has the widths of the benchmark model (Qwen3-8B: hidden 4096, 32 query heads on 8 KV heads
    # of 128, feed-forward 12288) with two layers and a small vocabulary, so that the plain
    # implementation can follow it in float64.  Its weights are made on the GPU (the same
    # values as on the host) and stored once, as bfloat16: the float32 path reads the same
    # values widened.
    "W": dict(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32,
              num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=2048,
              rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
              max_position_embeddings=4096, use_sliding_window=False, sliding_window=None,
              page_size=16, seed=8, stored="bfloat16", made_on="cuda:0"),
}
_NOT_CONFIG = ("page_size", "seed", "stored", "made_on")


def config_json(name: str, dtype: str = "float32") -> dict:
    c = {k: v for k, v in TINY[name].items() if k not in _NOT_CONFIG}
    c.update(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
             attention_bias=False, rope_scaling=None, torch_dtype=dtype)
    return c


_DIRS: Dict[tuple, str] = {}
_KEEP: List[tempfile.TemporaryDirectory] = []


def model_dir(name: str, dtype: str = "float32") -> str:
    """A temporary model folder (config.json + model.safetensors) with seeded random weights,
    written by the package's own random-weights mode."""
    dtype = TINY[name].get("stored", dtype)
    key = (name, dtype)
    if key not in _DIRS:
        from llmario_b200.config import Qwen3Config
        from llmario_b200.weights import write_random_model

        tmp = tempfile.TemporaryDirectory(prefix=f"llmario_tiny{name}_")
        _KEEP.append(tmp)
        cfg = Qwen3Config.from_dict(config_json(name, dtype))
        write_random_model(tmp.name, cfg, TINY[name]["seed"],
                           device=TINY[name].get("made_on", "cpu"))
        _DIRS[key] = tmp.name
    return _DIRS[key]


@functools.lru_cache(maxsize=None)
def _plain_model(name: str, dtype: str):
    return P.load(model_dir(name, dtype), torch.float64)


def plain_logits(name: str, dtype: str, tokens: Sequence[int], kv_round: Optional[str] = None
                 ) -> np.ndarray:
    """float64 logits [T, vocab] of the plain implementation on the stored weights."""
    tensors, cfg = _plain_model(name, TINY[name].get("stored", dtype))
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
#
# The bfloat16 figure is an upper bound for a deep model.  On the two-to-four-layer models of
# these tests the engine stays far below it, so each configuration is held to its own bound: the
# largest error seen over every replay mode, page size and kernel choice, times about two
# (BF16_BOUND, as a fraction of the largest logit; seen: A 0.0029, B 0.0076, C 0.0067, D 0.0075,
# E 0.0074, the seeded random configurations 0.0073 at most, W 0.012).  Split-K sums are added
# with atomics, so the last bits move from run to run; hence the factor.  A configuration
# without an entry is held to 2 %.
BF16_BOUND: Dict[str, float] = {"A": 8e-3, "B": 1.6e-2, "C": 1.5e-2, "D": 1.6e-2, "E": 1.6e-2,
                                "W": 2.5e-2}
BF16_DEFAULT_BOUND = 2e-2


def tolerance(dtype: str, ref: np.ndarray, name: Optional[str] = None) -> float:
    scale = max(1.0, float(np.abs(ref).max()))
    if dtype == "float32":
        return 1e-4 * scale
    return BF16_BOUND.get(name, BF16_DEFAULT_BOUND) * float(np.abs(ref).max())


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str = "",
                 name: Optional[str] = None) -> None:
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got.astype(np.float64) - ref)
    tol = tolerance(dtype, ref, name)
    log = os.environ.get("LLMARIO_TEST_ERROR_LOG")
    if log:      # one line per comparison: what, dtype, largest error as a fraction of the scale
        with open(log, "a") as f:
            f.write(f"{name or '-'}\t{dtype}\t{err.max() / max(1e-30, np.abs(ref).max()):.3e}"
                    f"\t{what}\n")
    worst = np.unravel_index(np.argmax(err), err.shape)
    assert err.max() <= tol, (f"{what}: max |diff| {err.max():.3e} > {tol:.3e} at row "
                              f"{worst[0]}, column {worst[1]}")


def check_greedy_against_plain(name: str, dtype: str, prompt: Sequence[int], out: Sequence[int],
                               what: str = "", margin: Optional[float] = None) -> int:
    """The plain implementation reads the engine's own sequence (prompt + generated tokens) and
    must choose the engine's token at every generated place where its two best logits are
    further apart than the engine's rounding can move them (``margin``, as a fraction of the
    largest logit).  Returns at how many places the choice was that clear."""
    if margin is None:
        margin = 1e-4 if dtype == "float32" else 2 * BF16_BOUND.get(name, BF16_DEFAULT_BOUND)
    ref = plain_logits(name, dtype, list(prompt) + list(out))
    clear = 0
    for j, tok in enumerate(out):
        l = ref[len(prompt) - 1 + j]
        top = np.sort(l)[-2:]
        if top[1] - top[0] > margin * max(1.0, float(np.abs(l).max())):
            clear += 1
            assert tok == int(np.argmax(l)), \
                f"{what}: token {j} is {tok}, the plain implementation chooses {int(np.argmax(l))}"
    return clear
