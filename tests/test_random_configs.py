"""Random configurations of the architecture (head sizes 32 to 128, one to eight query heads per
KV head, windows, pages of 8 to 64 positions, tied and untied heads) through random ways of
cutting a few requests, against the plain implementation.  The fixed tiny configurations pin
known corners; this sweeps the combinations between them, the same ones on every run."""
import random

import pytest

import traces
from test_replay import requests_for, run_in_process
from util import TINY

pytestmark = pytest.mark.gpu


def random_case(i: int):
    rng = random.Random(9000 + i)
    hd = rng.choice([64, 128, 128, 32])
    kvh = rng.choice([1, 2, 3])
    group = rng.choice([1, 2, 4, 8]) if hd != 32 else rng.choice([1, 2, 4])
    layers = rng.choice([1, 2, 3])
    window = rng.choice([None, None, rng.randrange(20, 200)])
    page = rng.choice([8, 16, 16, 32, 64])
    cfg = dict(num_hidden_layers=layers, hidden_size=rng.choice([64, 96, 136, 256]),
               num_attention_heads=kvh * group, num_key_value_heads=kvh, head_dim=hd,
               intermediate_size=rng.choice([96, 160, 264]), vocab_size=rng.choice([200, 333, 512]),
               rope_theta=rng.choice([1e4, 1e6]), rms_norm_eps=rng.choice([1e-6, 1e-5]),
               tie_word_embeddings=rng.random() < 0.5, max_position_embeddings=2048,
               use_sliding_window=window is not None, sliding_window=window, page_size=page,
               seed=i)
    if window is not None:
        cfg["layer_types"] = [rng.choice(["full_attention", "sliding_attention"])
                              for _ in range(layers)]
    lengths = tuple(rng.choice([1, 7, 33, 64, 65, 130, 257, 300, 420])
                    for _ in range(rng.randrange(3, 6)))
    mode = rng.choice(["mixed", "bulk_then_tail", "portions", "whole"])
    dtype = rng.choice(["bfloat16", "bfloat16", "float32"])
    return cfg, lengths, mode, dtype


@pytest.mark.parametrize("i", range(40))
def test_random_configuration(i):
    cfg, lengths, mode, dtype = random_case(i)
    name = f"R{i}"
    TINY[name] = cfg
    try:
        reqs = requests_for(name, lengths, seed=i)
        steps = (traces.mixed(reqs, live=4, seed=i) if mode == "mixed"
                 else getattr(traces, mode)(reqs))
        out, _ = run_in_process(name, dtype, steps, traces.peak_tokens(steps) + 64,
                                page=cfg["page_size"])
        what = (f"case {i}: head size {cfg['head_dim']}, {cfg['num_attention_heads']}/"
                f"{cfg['num_key_value_heads']} heads, window {cfg['sliding_window']}, page "
                f"{cfg['page_size']}, {mode}, {dtype}, lengths {lengths}")
        traces.check(steps, out, reqs, name, dtype, what)
    finally:
        del TINY[name]
