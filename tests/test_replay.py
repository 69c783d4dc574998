"""Replay of the same requests cut in different ways (whole; most at once and the last 32
tokens one by one; portions of changing size; mixed with other requests and so few pages that
they are used again), in 32-bit and in bfloat16, against the plain implementation."""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

import traces
from util import TINY, model_dir, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_in_process(name, dtype, steps, max_tokens, max_requests=8, page=None):
    """Drive the engine's own step function the way bin/trace_run does."""
    from llmario_b200.engine import Model, ModelRunner, StepEntry

    model = Model.from_folder(model_dir(name, dtype), dtype, "cuda:0")
    page = page or TINY[name]["page_size"]
    n_pages = -(-max_tokens // page)
    runner = ModelRunner(model, page_size=page, n_pages=n_pages, max_requests=max_requests,
                         max_context=min(model.spec.max_positions, n_pages * page))
    out = {}
    for s in steps:
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        if logits.shape[0]:
            out[s["step"]] = logits.cpu().numpy()
        for rid in s["end"]:
            runner.close(rid)
        runner.cache.check_invariants()
    assert not runner.cache.live_requests()
    assert all(f == n_pages for f in runner.cache.free_pages())
    return out, runner


def requests_for(name, lengths, seed):
    return {f"q{i}": random_tokens(name, n, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "bulk_then_tail", "portions"])
def test_one_request_at_a_time(name, dtype, mode):
    reqs = requests_for(name, (45, 97, 130) if name != "D" else (45, 170, 300), seed=7)
    steps = getattr(traces, mode)(reqs)
    out, _ = run_in_process(name, dtype, steps, traces.peak_tokens(steps))
    traces.check(steps, out, reqs, name, dtype, f"{name} {dtype} {mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_with_page_reuse(name, dtype):
    reqs = requests_for(name, (40, 23, 75, 7, 1, 110, 64, 33, 90), seed=11)
    steps = traces.mixed(reqs, live=4, seed=3)
    peak = traces.peak_tokens(steps)
    out, runner = run_in_process(name, dtype, steps, peak)
    traces.check(steps, out, reqs, name, dtype, f"{name} {dtype} mixed")
    page = TINY[name]["page_size"]
    total = sum(-(-len(t) // page) for t in reqs.values())
    # so few pages that they are used again: more were handed out than the pool holds
    assert runner.cache.counters["pages_allocated"] > runner.cache.groups[0].n_pages
    assert runner.cache.counters["pages_allocated"] >= total


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("D", 32), ("D", 64), ("A", 64), ("B", 64), ("C", 64)])
def test_larger_pages(name, page, dtype):
    """Pages of 32 and 64 positions (64 is what the engine and bin/trace_run use when they are
    not told a size).  With config D (head size 64, four heads per KV head, a window on one
    layer) in bfloat16 they are fetched by TMA in the attention of prompt portions and in decode
    attention; the other configurations take the kernels for other head sizes.  Portions of
    changing size, then a mixed batch with pages used again."""
    reqs = requests_for(name, (45, 170, 300) if name == "D" else (45, 97, 130), seed=7)
    steps = traces.portions(reqs)
    out, _ = run_in_process(name, dtype, steps, traces.peak_tokens(steps), page=page)
    traces.check(steps, out, reqs, name, dtype, f"{name} {dtype} portions, pages of {page}")
    reqs = requests_for(name, (40, 23, 75, 7, 1, 110, 64, 33, 90), seed=11)
    steps = traces.mixed(reqs, live=4, seed=3)
    out, runner = run_in_process(name, dtype, steps, traces.peak_tokens(steps), page=page)
    traces.check(steps, out, reqs, name, dtype, f"{name} {dtype} mixed, pages of {page}")
    assert runner.cache.counters["pages_allocated"] > runner.cache.groups[0].n_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_no_tensor_core_path_takes(dtype):
    """Config E: a width of 100, a feed-forward size of 76, five query heads on one KV head, a
    vocabulary of 333.  The products and the attention fall back to kernels that take these
    sizes; the logits are right all the same."""
    name = "E"
    reqs = requests_for(name, (45, 97, 130), seed=7)
    for mode in ("whole", "bulk_then_tail", "portions"):
        steps = getattr(traces, mode)(reqs)
        out, _ = run_in_process(name, dtype, steps, traces.peak_tokens(steps))
        traces.check(steps, out, reqs, name, dtype, f"{name} {dtype} {mode}")
    reqs = requests_for(name, (40, 23, 75, 7, 1, 110, 64, 33, 90), seed=11)
    steps = traces.mixed(reqs, live=4, seed=3)
    out, _ = run_in_process(name, dtype, steps, traces.peak_tokens(steps))
    traces.check(steps, out, reqs, name, dtype, f"{name} {dtype} mixed")


@pytest.mark.parametrize("name,dtype,mode", [("B", "float32", "mixed"), ("B", "bfloat16", "mixed"),
                                             ("D", "bfloat16", "mixed"),
                                             ("D", "bfloat16", "bulk_then_tail")])
def test_trace_run_program(name, dtype, mode):
    """The program itself: standard input to files, `done` lines, exit code.  It is run with
    the options the task gives it and nothing else, so its pages hold 64 positions."""
    if name == "B":
        reqs = requests_for(name, (50, 37, 20), seed=5)
    else:
        reqs = requests_for(name, (150, 260, 70, 33), seed=6)
    steps = traces.mixed(reqs, live=3, seed=1) if mode == "mixed" else getattr(traces, mode)(reqs)
    with tempfile.TemporaryDirectory() as out_dir:
        p = subprocess.run(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model",
             model_dir(name, dtype), "--dtype", dtype, "--out", out_dir, "--max-tokens",
             str(traces.peak_tokens(steps))],
            input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
            timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
        assert done == [f"done {s['step']}" for s in steps]
        vocab = TINY[name]["vocab_size"]
        out = {}
        for s in steps:
            path = os.path.join(out_dir, f"{s['step']}.f32")
            n = sum(len(e["want"]) for e in s["entries"])
            if n:
                out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n, vocab)
            else:
                assert not os.path.exists(path)
    traces.check(steps, out, reqs, name, dtype, f"trace_run {name} {dtype} {mode}")
