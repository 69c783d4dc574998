"""The native step driver against the same steps driven launch by launch from Python.

The driver (``csrc/step_driver.cu``) states the dispatch rules of ``llmario_b200.kernels`` a second
time, in C++.  The policies must give the same numbers, and whole steps the same logits: bit for
bit in 32-bit (no atomics, the same launches), within rounding in bfloat16 (split-K sums are
added with atomics), and the same as the plain implementation either way."""
import random

import numpy as np
import pytest
import torch

import traces
from util import model_dir, random_tokens


def test_native_policies_equal_the_python_ones():
    from llmario_b200 import kernels
    from llmario_b200.engine import native

    token_tile, k_splits, decode_splits = native.policies()
    for rows in (1, 2, 8, 16, 17, 32, 33, 64, 65, 128, 129, 300, 511, 512, 513, 2048, 5000):
        assert token_tile(rows) == kernels.token_tile(rows)
        for n, k in ((6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288), (151936, 4096),
                     (2048, 1024), (768, 256), (96, 64), (3072, 1024), (1024, 3072), (333, 100),
                     (10240, 5120), (51200, 5120), (5120, 25600)):
            assert k_splits(rows, n, k) == kernels.k_splits(rows, n, k), (rows, n, k)
    rng = random.Random(0)
    cases = [(n, kv, length, res, tile) for n in (1, 3, 8, 32, 64, 72, 300, 512) for kv in (1, 2, 8)
             for length in (1, 63, 64, 100, 128, 1024, 1100, 4096, 8192, 40000)
             for res, tile in ((444, 64), (888, 32), (444, 32))]
    cases += [(rng.randint(1, 600), rng.randint(1, 16), rng.randint(1, 50000),
               rng.choice((444, 888, 300)), rng.choice((32, 64))) for _ in range(500)]
    for c in cases:
        assert decode_splits(*c) == kernels.decode_splits(*c), c


def _replay(name, dtype, steps, max_tokens, page, use_native):
    from llmario_b200 import driver
    from llmario_b200.engine import Model, ModelRunner, StepEntry

    model = Model.from_folder(model_dir(name, dtype), dtype, "cuda:0")
    n_pages = -(-max_tokens // page)
    runner = ModelRunner(model, page_size=page, n_pages=n_pages, max_requests=8,
                         max_context=min(model.spec.max_positions, n_pages * page),
                         use_native=use_native)
    assert (runner.native is not None) == use_native
    out = {}
    for s in steps:
        if use_native and s["step"] % 3 == 0:
            driver.arena_fill(0xFF)      # stale scratch contents must not reach any result
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        if logits.shape[0]:
            out[s["step"]] = logits.cpu().numpy()
        for rid in s["end"]:
            runner.close(rid)
    return out, runner


@pytest.mark.gpu
@pytest.mark.parametrize("name,dtype,page", [("A", "float32", 4), ("B", "float32", 8),
                                             ("C", "float32", 16), ("D", "float32", 16),
                                             ("E", "float32", 8), ("D", "bfloat16", 16),
                                             ("D", "bfloat16", 64), ("B", "bfloat16", 8),
                                             ("C", "bfloat16", 16), ("E", "bfloat16", 8),
                                             ("W", "bfloat16", 16)])
def test_native_and_python_driven_steps_agree(name, dtype, page):
    """Mixed batches with pages used again, then each request most at once and its tail token
    by token (recorded steps), both ways."""
    lengths = (40, 23, 75, 7, 1, 110, 64, 33, 90) if name != "W" else (40, 23, 75, 7, 1, 110)
    reqs = {f"q{i}": random_tokens(name, n, 11 + i) for i, n in enumerate(lengths)}
    for steps in (traces.mixed(reqs, live=4, seed=3), traces.bulk_then_tail(dict(list(reqs.items())[:3]))):
        peak = traces.peak_tokens(steps)
        py, _ = _replay(name, dtype, steps, peak, page, use_native=False)
        nat, runner = _replay(name, dtype, steps, peak, page, use_native=True)
        assert py.keys() == nat.keys()
        for k in py:
            if dtype == "float32":
                assert np.array_equal(py[k], nat[k]), (name, k)
            else:
                scale = np.abs(py[k]).max()
                assert np.abs(py[k] - nat[k]).max() <= 1e-2 * scale, (name, k)
        traces.check(steps, nat, {r: reqs[r] for s in steps for e in s["entries"]
                                  for r in [e["id"]]}, name, dtype, f"native {name} {dtype}")
    assert runner.counters["graph_replays"] > 0


@pytest.mark.gpu
def test_many_requests_with_few_pages_native_or_not():
    """Requests that wait, run beside prompt portions, are preempted and recomputed: the tokens
    are the same whether the layers are driven natively or from Python."""
    from llmario_b200 import Engine, SamplingParams
    name, dtype = "D", "float32"
    rng = random.Random(5)
    prompts = [random_tokens(name, rng.randint(3, 90), 300 + i) for i in range(40)]
    params = [SamplingParams(temperature=0.0 if i % 3 else 0.9, seed=100 + i,
                             max_tokens=rng.randint(4, 60)) for i in range(40)]

    def run(native):
        eng = Engine(model_dir(name, dtype), dtype=dtype, page_size=16, cache_tokens=352,
                     max_requests=6, context=256, token_budget=48, native=native)
        outs = eng.generate(prompts, params)
        assert (eng.runner.native is not None) == native
        return outs, eng.stats()

    a, st_a = run(False)
    b, st_b = run(True)
    assert a == b and st_b["preemptions"] > 0
    assert st_a["steps"] == st_b["steps"]


@pytest.mark.gpu
def test_host_time_of_a_mixed_step():
    """The host's time to issue a mixed step of a 28-layer model of small widths (the sizes of
    the smallest benchmark configuration, a small vocabulary), native against Python-driven:
    measured around the step function without waiting for the device."""
    import time
    from llmario_b200.cli import preset_config
    from llmario_b200.config import Qwen3Config
    from llmario_b200.engine import Model, ModelRunner, StepEntry

    raw = dict(preset_config("qwen3-0.6b").to_dict(), vocab_size=4096, max_position_embeddings=4096)
    cfg = Qwen3Config.from_dict(raw)
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    rng = random.Random(0)
    times = {}
    for use_native in (False, True):
        runner = ModelRunner(model, page_size=16, cache_tokens=16384, max_requests=16,
                             max_context=2048, use_native=use_native)
        for r in range(8):
            runner.step([StepEntry(f"d{r}", [rng.randrange(4096) for _ in range(50 + r)], [])])
        best = None
        for it in range(6):
            entries = [StepEntry(f"d{r}", [rng.randrange(4096)], [0]) for r in range(8)]
            entries += [StepEntry(f"p{it}", [rng.randrange(4096) for _ in range(300)], [299])]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            runner.step(entries)
            dt = time.perf_counter() - t0
            torch.cuda.synchronize()
            runner.close(f"p{it}")
            if it >= 2:
                best = dt if best is None else min(best, dt)
        times[use_native] = best
    # (the driver takes out most of the time that Python spends on launches; what it leaves is the
    # CUDA driver's own time for some 230 launches and the step's bookkeeping)
    assert times[True] * 2 <= times[False], times
    print(f"host time of a mixed step: python {times[False] * 1e3:.2f} ms, "
          f"native {times[True] * 1e3:.2f} ms")
