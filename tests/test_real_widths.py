"""The widths of the benchmark model against the plain implementation.

Configuration W has the layer sizes that ``bench.py`` times (hidden 4096, 32 query heads on 8 KV
heads of 128, feed-forward 12288) with two layers and a vocabulary of 2,048, so that the plain
float64 implementation can follow it on the CPU.  At these widths the bfloat16 engine takes the
tcgen05 products (with split K for few rows, on CTA pairs for many), the tcgen05 attention of
prompt portions and the TMA decode attention; with many live requests decode attention splits
the keys and merges, with few it runs fused with the rotation and the cache write; steps of
single tokens are recorded as CUDA graphs, one per context bucket.  Every cut of the work, in
32-bit and in bfloat16, with pages of 16 and of 64 positions, is compared with the plain logits.
"""
import random

import numpy as np
import pytest

import traces
from test_replay import requests_for, run_in_process
from util import assert_close, model_dir, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAME = "W"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [16, 64])
def test_every_cut_at_benchmark_widths(dtype, page):
    reqs = requests_for(NAME, (45, 170, 300), seed=7)
    for mode in ("whole", "bulk_then_tail", "portions"):
        steps = getattr(traces, mode)(reqs)
        out, _ = run_in_process(NAME, dtype, steps, traces.peak_tokens(steps), page=page)
        traces.check(steps, out, reqs, NAME, dtype, f"W {dtype} {mode}, pages of {page}")
    reqs = requests_for(NAME, (40, 23, 75, 7, 1, 110, 64, 33, 90), seed=11)
    steps = traces.mixed(reqs, live=4, seed=3)
    out, runner = run_in_process(NAME, dtype, steps, traces.peak_tokens(steps), page=page)
    traces.check(steps, out, reqs, NAME, dtype, f"W {dtype} mixed, pages of {page}")
    assert runner.cache.counters["pages_allocated"] > runner.cache.groups[0].n_pages


@pytest.mark.parametrize("dtype,live,mode", [("float32", 72, "default"), ("bfloat16", 72, "default"),
                                             ("bfloat16", 80, "separate"),
                                             ("bfloat16", 80, "persistent"),
                                             ("float32", 8, "default"), ("bfloat16", 8, "default")])
def test_many_live_requests_decode_through_recorded_steps(dtype, live, mode):
    """``live`` requests with prompts of unequal length, then 44 steps of one token each.  Many
    requests share a length modulo the page size, so their block tables change in the same
    step; the context bucket of the recorded step changes on the way (positions cross 128).
    In bfloat16 the rows of a step fit two waves of the fused decode kernel (norm, rotation,
    cache write and attention in one); ``separate`` keeps the rotation kernel and the decode
    attention apart, as steps of more rows run, and ``persistent`` takes the persistent decode
    kernel with its merge there.  Every row of every step against the plain implementation."""
    from llmario_b200 import driver, kernels

    driver.use_persistent_decode(mode == "persistent")
    kernels.fuse_decode("few waves" if mode == "default" else "never")
    try:
        _many_live(dtype, live, mode)
    finally:
        driver.use_persistent_decode(False)
        kernels.fuse_decode("few waves")


def _many_live(dtype, live, mode):
    from llmario_b200 import kernels
    from llmario_b200.engine import Model, ModelRunner, StepEntry

    page, steps = 16, 44
    rng = random.Random(live)
    # lengths: a third end just before a page edge, so that their first decode steps all open a
    # new page together; the rest spread out, a few long enough to start beyond position 128
    lengths = [(15, 31, 47)[i % 3] if i % 3 == 0 else rng.randint(3, 60) for i in range(live)]
    for i in range(0, live, 9):
        lengths[i] = rng.randint(100, 120)
    prompts = {f"r{i}": random_tokens(NAME, n, 500 + i) for i, n in enumerate(lengths)}
    tails = {r: random_tokens(NAME, steps, 900 + i) for i, r in enumerate(prompts)}
    model = Model.from_folder(model_dir(NAME, dtype), dtype, DEV)
    cache_tokens = sum(-(-(n + steps) // page) * page for n in lengths) + page
    runner = ModelRunner(model, page_size=page, cache_tokens=cache_tokens, max_requests=live,
                         max_context=256, token_budget=1024)
    from llmario_b200.engine import native
    # the layers are driven natively: the driver counts which kernels it chose
    assert runner.native is not None
    ids = list(prompts)
    got = {r: [] for r in ids}
    at = 0
    while at < live:                     # prompts, several to a step, under the token budget
        batch, rows = [], 0
        while at < live and rows + lengths[at] <= 1024 and len(batch) < 16:
            batch.append(ids[at])
            rows += lengths[at]
            at += 1
        res = runner.step([StepEntry(r, prompts[r], [len(prompts[r]) - 1]) for r in batch])
        for j, r in enumerate(batch):
            got[r].append(res[j:j + 1].cpu().numpy())
    before = native.kernel_counts()
    crossings = 0
    for s in range(steps):
        crossings = max(crossings, sum((lengths[i] + s) % page == 0 for i in range(live)))
        res = runner.step([StepEntry(r, [tails[r][s]], [0]) for r in ids]).cpu().numpy()
        for j, r in enumerate(ids):
            got[r].append(res[j:j + 1])
        runner.cache.check_invariants()
    kernels.check_tc_status(DEV)
    assert crossings >= max(2, live // 5)       # that many requests opened a page in one step
    c = runner.counters
    assert c["graphs_recorded"] >= 2 and c["graph_replays"] >= steps - 6, c
    if dtype == "bfloat16":
        after = native.kernel_counts()
        fused = after["decode_fused"] - before["decode_fused"]
        split = after["decode_tma"] + after["decode_persistent"] - before["decode_tma"] - \
            before["decode_persistent"]
        if mode == "default":
            assert fused > 0 and split == 0
        else:
            assert fused == 0 and split > 0 and after["rope_store"] > before["rope_store"]
            assert (after["decode_persistent"] > before["decode_persistent"]) == (mode == "persistent")
            if mode == "persistent":
                assert after["merge"] > before["merge"]
        assert after["gemm_tcgen05"] > before["gemm_tcgen05"] and after["gemm_simt"] == before["gemm_simt"]
    for r in ids:
        ref = plain_logits(NAME, dtype, prompts[r] + tails[r])
        rows = np.concatenate(got[r])
        assert_close(rows, ref[len(prompts[r]) - 1:len(prompts[r]) + steps], dtype,
                     f"W {dtype} {live} live, {r}", NAME)
    for r in ids:
        runner.close(r)
    assert all(f == runner.cache.groups[0].n_pages for f in runner.cache.free_pages())


@pytest.mark.parametrize("lookahead", [False, True])
def test_generation_with_many_requests_at_benchmark_widths(lookahead):
    """Greedy generation of 72 requests through the entry point in bfloat16, with and without
    the next step queued ahead: for a sample of the requests the plain implementation reads the
    engine's own sequence and must choose the same token at every place where its two best
    logits are further apart than the engine's rounding."""
    from llmario_b200 import Engine, SamplingParams

    live, new = 72, 40
    rng = random.Random(3)
    prompts = [random_tokens(NAME, rng.randint(3, 70), 700 + i) for i in range(live)]
    eng = Engine(model_dir(NAME, "bfloat16"), dtype="bfloat16", page_size=16,
                 cache_tokens=live * 128, max_requests=live, context=256, token_budget=512,
                 lookahead=lookahead)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    st = eng.stats()
    assert st["finished"] == live and st["graph_replays"] >= new // 2
    assert (st["steps_planned_ahead"] > new // 2) == lookahead
    assert st["free_pages"] == st["pages"] and st["failed_steps"] == 0
    for i in range(0, live, 6):
        assert len(outs[i]) == new
        ref = plain_logits(NAME, "bfloat16", prompts[i] + outs[i])
        for j, tok in enumerate(outs[i]):
            l = ref[len(prompts[i]) - 1 + j]
            top = np.sort(l)[-2:]
            if top[1] - top[0] > 3e-2 * max(1.0, float(np.abs(l).max())):
                assert tok == int(np.argmax(l)), (i, j, tok, int(np.argmax(l)))


def test_long_portion_with_two_query_tiles_per_cta():
    """A prompt portion long enough for the attention kernel with two query tiles per CTA (pages
    of 32 positions, where the driver chooses it), then a portion that continues the request
    with the one-tile kernel: logits at several places against the plain implementation."""
    from llmario_b200 import kernels
    from llmario_b200.engine import Model, ModelRunner, StepEntry, native

    toks = random_tokens(NAME, 2400 + 150, 77)
    want = [0, 63, 64, 1000, 2047, 2399]
    model = Model.from_folder(model_dir(NAME, "bfloat16"), "bfloat16", DEV)
    runner = ModelRunner(model, page_size=32, cache_tokens=4096, max_requests=2, max_context=4096,
                         token_budget=4096)
    before = native.kernel_counts()
    a = runner.step([StepEntry("r", toks[:2400], want)]).float().cpu().numpy()
    mid = native.kernel_counts()
    b = runner.step([StepEntry("r", toks[2400:], [0, 77, 149])]).float().cpu().numpy()
    after = native.kernel_counts()
    kernels.check_tc_status(DEV)
    assert mid["tcgen05_x2"] - before["tcgen05_x2"] == 2           # both layers
    assert after["tcgen05_x2"] == mid["tcgen05_x2"] and after["tcgen05"] - mid["tcgen05"] == 2
    ref = plain_logits(NAME, "bfloat16", toks)
    assert_close(a, ref[want], "bfloat16", "two query tiles per CTA", NAME)
    assert_close(b, ref[[2400, 2477, 2549]], "bfloat16", "continued with one tile", NAME)


@pytest.mark.parametrize("page", [8, 16])
def test_long_portions_over_small_pages_read_gathered_keys(page):
    """With pages too small for TMA boxes, portions of many tokens read a gathered copy of
    their requests' keys and values; short portions in the same step read the cache as it is.
    A request is cut into portions so that later portions gather what earlier steps wrote;
    against the plain implementation, and against the same steps without gathering."""
    from llmario_b200 import driver, kernels
    from llmario_b200.engine import Model, ModelRunner, StepEntry, native

    reqs = {"a": random_tokens(NAME, 700, 31), "b": random_tokens(NAME, 333, 32),
            "c": random_tokens(NAME, 60, 33)}
    plan = [[("a", 0, 300), ("c", 0, 40)], [("a", 300, 200), ("b", 0, 333), ("c", 40, 1)],
            [("a", 500, 200), ("c", 41, 19)]]
    model = Model.from_folder(model_dir(NAME, "bfloat16"), "bfloat16", DEV)
    outs = {}
    for gather in (True, False):
        driver.use_gather(gather)
        try:
            runner = ModelRunner(model, page_size=page, cache_tokens=2048, max_requests=4,
                                 max_context=1024, token_budget=1024)
            before = native.kernel_counts()
            got = {r: [] for r in reqs}
            for step in plan:
                # what the driver's scratch buffers hold from earlier steps must not matter:
                # every value in them is made a NaN
                driver.arena_fill(0xFF)
                res = runner.step([StepEntry(r, reqs[r][s:s + n], list(range(n)))
                                   for r, s, n in step]).float().cpu().numpy()
                at = 0
                for r, s, n in step:
                    got[r].append(res[at:at + n])
                    at += n
            kernels.check_tc_status(DEV)
            after = native.kernel_counts()
            # two layers, three steps; portions of 128 tokens or more are gathered
            assert (after["kv_gather"] - before["kv_gather"] == 6) == gather
            outs[gather] = {r: np.concatenate(v) for r, v in got.items()}
        finally:
            driver.use_gather(True)
    for r, toks in reqs.items():
        ref = plain_logits(NAME, "bfloat16", toks)
        assert_close(outs[True][r], ref, "bfloat16", f"gathered keys, pages of {page}, {r}", NAME)
        assert_close(outs[False][r], ref, "bfloat16", f"cache as it is, pages of {page}, {r}", NAME)
