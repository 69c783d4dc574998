"""The engine through its entry point, the sampler on the device, the parts alone, and parts
defined by a test."""
import dataclasses
import random

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P
from util import (TINY, assert_close, check_greedy_against_plain, model_dir,
                  plain_logits, random_tokens)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def plain_greedy(name, dtype, prompt, n, margin):
    """Greedy continuation by the plain implementation; also says at which steps its two best
    logits are closer than ``margin`` (there the engine's rounding may pick the other)."""
    seq, out, close = list(prompt), [], []
    for _ in range(n):
        l = plain_logits(name, dtype, seq)[-1]
        top = np.sort(l)[-2:]
        close.append(top[1] - top[0] <= margin * max(1.0, np.abs(l).max()))
        out.append(int(np.argmax(l)))
        seq.append(out[-1])
    return out, close


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_greedy_generation_through_the_entry_point(name, dtype):
    from llmario_b200 import Engine, SamplingParams
    eng = Engine(model_dir(name, dtype), dtype=dtype, page_size=TINY[name]["page_size"],
                 cache_tokens=512, max_requests=4, context=256, token_budget=16)
    prompts = [random_tokens(name, n, 40 + n) for n in (5, 11, 17)]      # the workload of config A
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    margin = 1e-4 if dtype == "float32" else 3e-2
    for prompt, out in zip(prompts, outs):
        assert len(out) == 8
        want, close = plain_greedy(name, dtype, prompt, 8, margin)
        for i, (a, b) in enumerate(zip(out, want)):
            if close[i]:
                break            # a near-tie: later tokens may legitimately differ
            assert a == b, f"{name} {dtype}: token {i} is {a}, plain {b}"
    st = eng.stats()
    assert st["finished"] == 3 and st["free_pages"] == st["pages"]
    assert st["max_entries_in_step"] >= 2            # requests shared steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype):
    """300 tokens one by one from an empty cache (first tokens included) against the whole."""
    from llmario_b200.engine import Model, ModelRunner, StepEntry
    name = "C"
    toks = random_tokens(name, 300, 9)
    model = Model.from_folder(model_dir(name, dtype), dtype, DEV)
    runner = ModelRunner(model, page_size=16, n_pages=20, max_requests=2, max_context=320)
    rows = [runner.step([StepEntry("r", [t], [0])])[0].cpu().numpy() for t in toks]
    assert_close(np.stack(rows), plain_logits(name, dtype, toks), dtype, f"long decode {dtype}", name)


def test_float32_weights_stay_float32_in_bfloat16_mode():
    """A folder stored in 32-bit, run with --dtype bfloat16: the matrices stay 32-bit and the
    result is closer to the plain implementation than bfloat16 weights would allow."""
    from llmario_b200.engine import Model, ModelRunner, StepEntry
    name = "B"
    model = Model.from_folder(model_dir(name, "float32"), "bfloat16", DEV)
    assert model.blocks[0].mixer.o_proj.weight.dtype == torch.float32
    runner = ModelRunner(model, page_size=8, n_pages=16, max_requests=2, max_context=128)
    toks = random_tokens(name, 50, 3)
    got = runner.step([StepEntry("r", toks, list(range(50)))]).cpu().numpy()
    assert_close(got, plain_logits(name, "float32", toks), "bfloat16", "f32 weights, bf16 mode", name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_twice_and_shared_cache(dtype):
    """The order of layers is data: a layer run twice (own cache each time) and a call that
    reads an earlier call's cache, against the plain implementation with the same order."""
    from llmario_b200.config import LayerCall, load_spec
    from llmario_b200.engine import Model, ModelRunner, StepEntry
    name = "A"
    d = model_dir(name, dtype)
    spec = load_spec(d)
    order = (LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(0, reads_cache_of=1))
    model = Model.from_folder(d, dtype, DEV, spec=dataclasses.replace(spec, run_order=order))
    runner = ModelRunner(model, page_size=4, n_pages=64, max_requests=2, max_context=128)
    assert len(runner.cache.groups) == 1 and len(runner.cache.groups[0].entries) == 3
    toks = random_tokens(name, 37, 4)
    tensors, cfg = P.load(d)
    ref = P.forward_logits(tensors, cfg, toks, schedule=[(0, None), (1, None), (1, None), (0, 1)]).numpy()
    got = [runner.step([StepEntry("r", toks[:20], list(range(20)))]).cpu().numpy()]
    got += [runner.step([StepEntry("r", [t], [0])]).cpu().numpy() for t in toks[20:]]
    assert_close(np.concatenate(got), ref, dtype, f"run order {dtype}")


# ----------------------------------------------------------------------------- sampler
def test_device_sampler_matches_plain_chain():
    from llmario_b200.sampling import DeviceSampler, RequestSampler, SamplingParams
    rng = random.Random(0)
    V = 1000
    g = torch.Generator().manual_seed(0)
    sampler = DeviceSampler(DEV)
    cases = [dict(temperature=0.0), dict(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0),
             dict(temperature=0.7, top_k=0, top_p=1.0, min_p=0.0),
             dict(temperature=0.7, top_k=40, top_p=1.0, min_p=0.0),
             dict(temperature=1.3, top_k=5, top_p=0.8, min_p=0.0),
             dict(temperature=1.0, top_k=0, top_p=0.9, min_p=0.0),
             dict(temperature=0.8, top_k=0, top_p=1.0, min_p=0.1),
             dict(),                                  # the defaults: 40 / 0.95 / 0.05
             dict(temperature=1.0, top_k=1), dict(temperature=2.0, top_k=V + 5, top_p=0.5)]
    for trial in range(6):
        logits = (3.0 * torch.randn(len(cases), V, generator=g)).float()
        logits[:, 17] = logits[:, 400] = logits.max() + 0.5        # a tie at the top
        rs = []
        for c in cases:
            r = RequestSampler(SamplingParams(seed=trial * 100 + len(rs), **c), V)
            rs.append(r)
        twins = [P.PlainRng(r.seed) for r in rs]
        got = sampler.sample(logits.to(DEV), rs)
        for i, c in enumerate(cases):
            p = SamplingParams(**c)
            u = 0.0 if p.greedy else twins[i].next_f64()
            want = P.plain_sample(logits[i].tolist(), temperature=p.temperature, top_k=p.top_k,
                                  top_p=p.top_p, min_p=p.min_p, u=u)
            assert got[i] == want, (trial, c, u)


def test_device_sampler_penalties_and_streams():
    from llmario_b200.sampling import DeviceSampler, RequestSampler, SamplingParams
    V = 64
    logits = torch.zeros(2, V)
    logits[:, 3], logits[:, 9] = 5.0, 4.9
    pen = RequestSampler(SamplingParams(temperature=0, repeat_penalty=1.5), V)
    pen.accept(3)
    plain = RequestSampler(SamplingParams(temperature=0), V)
    assert DeviceSampler(DEV).sample(logits.to(DEV), [pen, plain]) == [9, 3]
    freq = RequestSampler(SamplingParams(temperature=0, frequency_penalty=0.06,
                                         presence_penalty=0.0, repeat_last_n=2), V)
    for t in (3, 3, 3):
        freq.accept(t)                       # window of 2: count 2 -> 5.0 - 0.12 < 4.9
    assert list(freq.window) == [3, 3] and freq.counts == {3: 2}
    assert DeviceSampler(DEV).sample(logits[:1].to(DEV), [freq]) == [9]
    # a seed gives the same tokens whatever else is in the batch; frequencies follow the softmax
    l = torch.log(torch.tensor([0.5, 0.3, 0.2] + [1e-9] * (V - 3)))[None, :]
    params = SamplingParams(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=7)
    a = RequestSampler(params, V)
    alone = [DeviceSampler(DEV).sample(l.to(DEV), [a])[0] for _ in range(300)]
    b = RequestSampler(params, V)
    other = RequestSampler(SamplingParams(temperature=0.9, seed=1), V)
    mixed = [DeviceSampler(DEV).sample(l.repeat(2, 1).to(DEV), [other, b])[1] for _ in range(300)]
    assert alone == mixed
    freqs = [alone.count(i) / 300 for i in range(3)]
    assert abs(freqs[0] - 0.5) < 0.09 and abs(freqs[1] - 0.3) < 0.09 and abs(freqs[2] - 0.2) < 0.08


def test_penalties_count_a_token_in_flight():
    """A step queued ahead draws with penalties while the token that just entered the window is
    still on the device: the sampler gets the counts without that token and the row of the draw
    before that holds it.  The penalised logits and the drawn tokens must be, bit for bit, those
    of a draw that had the token on the host: when the token is already in the window, when it
    is new to it, and when the window is full and its oldest token leaves as the new one comes."""
    from llmario_b200 import SamplingParams
    from llmario_b200.sampling import DeviceSampler, RequestSampler

    vocab, rows = 257, 5
    gen = torch.Generator().manual_seed(3)
    base = (3.0 * torch.randn(rows, vocab, generator=gen)).to(DEV)
    params = [SamplingParams(temperature=0.0, repeat_penalty=1.3, frequency_penalty=0.4,
                             presence_penalty=0.2, repeat_last_n=6),
              SamplingParams(temperature=0.8, top_k=0, top_p=1.0, min_p=0.0, seed=5,
                             repeat_penalty=1.2, frequency_penalty=0.3, repeat_last_n=6),
              SamplingParams(temperature=0.0),                       # no penalties on this row
              SamplingParams(temperature=0.0, repeat_penalty=1.5, repeat_last_n=4),
              SamplingParams(temperature=0.0, frequency_penalty=0.7, repeat_last_n=64)]
    histories = [[7, 9, 7], [1, 2, 3, 4, 5, 6], [4, 4], [8, 9, 10, 11], [20, 21]]
    new = [7, 99, 4, 8, 21]           # in the window / new to it / (no penalties) / the one that leaves / in it

    def samplers():
        out = []
        for p, h in zip(params, histories):
            s = RequestSampler(p, vocab)
            for t in h:
                s.accept(t)
            out.append(s)
        return out

    # the draw before: its tokens lie in the sampler's device buffer (rows in another order)
    order = [3, 0, 4, 1, 2]
    dev = DeviceSampler(DEV)
    want_rows = torch.full((rows, vocab), -50.0, device=DEV)
    for j, r in enumerate(order):
        want_rows[j, new[r]] = 50.0
    assert dev.sample(want_rows, [RequestSampler(SamplingParams(temperature=0.0), vocab)
                                  for _ in range(rows)]) == [new[r] for r in order]
    ahead = samplers()
    la = base.clone()
    got_ahead = dev.launch(la, ahead, inflight=[order.index(r) for r in range(rows)]).result()
    # the same draw with the tokens known on the host
    known = samplers()
    for s, t in zip(known, new):
        s.accept(t)
    lk = base.clone()
    got_known = DeviceSampler(DEV).sample(lk, known)
    assert torch.equal(la, lk) and got_ahead == got_known
    assert not torch.equal(la, base) and torch.equal(la[2], base[2])


def test_temperature_generation_is_reproducible_and_batch_independent():
    """Config B's workload: four requests of 1/7/23/40 tokens, prompts cut at 16 beside
    running decodes, 12 tokens at temperature 0.7 with a seed."""
    from llmario_b200 import Engine, SamplingParams
    name, dtype = "B", "float32"
    prompts = [random_tokens(name, n, 70 + n) for n in (1, 7, 23, 40)]
    params = [SamplingParams(temperature=0.7, seed=11 + i, max_tokens=12) for i in range(4)]

    def run(order, budget):
        eng = Engine(model_dir(name, dtype), dtype=dtype, page_size=8, cache_tokens=512,
                     max_requests=4, context=128, token_budget=budget)
        outs = eng.generate([prompts[i] for i in order], [params[i] for i in order])
        return {i: o for i, o in zip(order, outs)}

    a = run([0, 1, 2, 3], 16)
    b = run([3, 2, 1, 0], 64)
    alone = {i: run([i], 16)[i] for i in range(4)}
    assert all(len(a[i]) == 12 for i in range(4))
    assert a == alone            # same seed, same logits (to rounding) -> same tokens
    assert a == b


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_queued_ahead_give_the_same_tokens(dtype):
    """With a step queued while the one before it still runs (its input tokens taken from the
    sampler's output on the device), the engine returns what it returns step by step: greedy
    and seeded temperature sampling, different lengths, an end-of-sequence token in the middle
    of one request, and a request that joins later."""
    from llmario_b200 import Engine, SamplingParams
    name = "D"
    prompts = [random_tokens(name, n, 90 + n) for n in (3, 19, 33, 6)]
    params = [SamplingParams(temperature=0.0, max_tokens=40),
              SamplingParams(temperature=0.8, seed=5, max_tokens=25),
              SamplingParams(temperature=0.0, max_tokens=9),
              SamplingParams(temperature=0.6, seed=9, max_tokens=30)]

    def run(lookahead, eos=()):
        eng = Engine(model_dir(name, dtype), dtype=dtype, page_size=16, cache_tokens=1024,
                     max_requests=4, context=256, token_budget=32, lookahead=lookahead)
        eng.scheduler.eos = frozenset(eos)
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts[:3], params[:3])]
        for _ in range(6):
            eng.step()
        ids.append(eng.add_request(prompts[3], params[3]))      # joins while the others decode
        eng.run_until_done()
        assert min(eng.runner.cache.free_pages()) == eng.runner.cache.groups[0].n_pages
        eng.runner.cache.check_invariants()
        return [(list(eng.request(i).output), eng.request(i).finish_reason) for i in ids], \
            eng.stats()

    if dtype == "bfloat16":
        # 16-bit sums of split products are added with atomics, so logits differ in their last
        # bits from run to run and a draw near a boundary may fall either way: here every
        # request is greedy and each run is held to the plain implementation instead
        params = [SamplingParams(temperature=0.0, max_tokens=p.max_tokens) for p in params]
        for lookahead in (False, True):
            res, stats = run(lookahead)
            clear = 0
            for prompt, (out, reason), p in zip(prompts, res, params):
                assert len(out) == p.max_tokens and reason == "length"
                clear += check_greedy_against_plain(name, dtype, prompt, out,
                                                    f"lookahead {lookahead}")
            assert clear >= 20
            assert (stats.get("steps_planned_ahead", 0) >= 20) == lookahead
        return
    plain_run, _ = run(False)
    ahead_run, stats = run(True)
    assert ahead_run == plain_run
    assert stats.get("steps_planned_ahead", 0) >= 20          # and most steps were queued ahead
    eos = plain_run[0][0][17]               # the first request now stops at its 18th token
    stop_plain, _ = run(False, [eos])
    stop_ahead, _ = run(True, [eos])
    assert stop_ahead == stop_plain
    first = stop_plain[0][0]
    assert stop_plain[0][1] == "stop" and first[-1] == eos and len(first) <= 18


def test_many_requests_with_few_pages_give_the_same_tokens_either_way():
    """Forty requests of mixed lengths through a cache that holds a fraction of them, so that
    requests wait, run beside prompt portions, are preempted and recomputed: with and without a
    step queued ahead the generated tokens are the same, every page comes back, and steps were
    in fact queued ahead and requests in fact preempted."""
    from llmario_b200 import Engine, SamplingParams
    name, dtype = "D", "float32"
    rng = random.Random(5)
    prompts = [random_tokens(name, rng.randint(3, 90), 300 + i) for i in range(40)]
    params = [SamplingParams(temperature=0.0 if i % 3 else 0.9, seed=100 + i,
                             max_tokens=rng.randint(4, 60)) for i in range(40)]

    def run(lookahead):
        eng = Engine(model_dir(name, dtype), dtype=dtype, page_size=16, cache_tokens=352,
                     max_requests=6, context=256, token_budget=48, lookahead=lookahead)
        outs = eng.generate(prompts, params)
        cache = eng.runner.cache
        cache.check_invariants()
        assert min(cache.free_pages()) == cache.groups[0].n_pages and not cache.live_requests()
        return outs, eng.stats()

    plain_run, st0 = run(False)
    ahead_run, st1 = run(True)
    assert ahead_run == plain_run
    assert [len(o) for o in plain_run] == [p.max_tokens for p in params]
    assert st1.get("steps_planned_ahead", 0) > 10 and st0["preemptions"] > 0 and st1["preemptions"] > 0


@pytest.mark.parametrize("every,cache_tokens", [(2, 400), (8, 400), (12, 2048)])
def test_requests_arrive_and_are_aborted_while_others_run(every, cache_tokens):
    """Requests arrive over time (one in ``every`` iterations), a few are aborted at random
    moments (also while a step that was queued ahead is in flight), the sampling options are
    mixed, and with the small cache requests are preempted.  Every request that was not aborted
    gets the tokens it gets alone in an engine of its own; no page is lost on the way."""
    from llmario_b200 import Engine, SamplingParams
    name, dtype, n = "D", "float32", 90
    rng = random.Random(every * 1000 + cache_tokens)
    prompts = [random_tokens(name, rng.randint(1, 140), 5000 + i) for i in range(n)]
    params = [SamplingParams(temperature=0.0 if rng.random() < 0.6 else rng.choice([0.5, 1.0, 1.3]),
                             top_k=rng.choice([0, 5, 40]), top_p=rng.choice([1.0, 0.9]),
                             min_p=rng.choice([0.0, 0.05]), seed=900 + i,
                             repeat_penalty=rng.choice([1.0, 1.1]),
                             frequency_penalty=rng.choice([0.0, 0.2]),
                             max_tokens=rng.randint(1, 70)) for i in range(n)]
    eng = Engine(model_dir(name, dtype), dtype=dtype, page_size=16, cache_tokens=cache_tokens,
                 max_requests=6, context=256, token_budget=48, lookahead=True)
    ids, aborted, nxt, steps = {}, set(), 0, 0
    while nxt < n or eng.has_work():
        if nxt < n and rng.random() < 1.0 / every:
            ids[nxt] = eng.add_request(prompts[nxt], params[nxt])
            nxt += 1
        if eng.has_work():
            eng.step()
            steps += 1
        if ids and rng.random() < 0.04:
            k = rng.choice(list(ids))
            if eng.request(ids[k]).finish_reason is None:
                eng.abort(ids[k])
                aborted.add(k)
        if steps % 64 == 0:
            eng.runner.cache.check_invariants()
    cache, st = eng.runner.cache, eng.stats()
    cache.check_invariants()
    assert min(cache.free_pages()) == cache.groups[0].n_pages and not cache.live_requests()
    assert st["failed_steps"] == 0 and aborted and len(aborted) < n // 2
    if cache_tokens < 1000:
        assert st["preemptions"] > 0
    if every >= 8:
        assert st["steps_planned_ahead"] > 0
    alone = Engine(model_dir(name, dtype), dtype=dtype, page_size=16, cache_tokens=1024,
                   max_requests=2, context=256, token_budget=256, lookahead=False)
    for k in range(n):
        r = eng.request(ids[k])
        if k in aborted:
            assert r.finish_reason == "aborted"
            continue
        assert r.finish_reason == "length" and len(r.output) == params[k].max_tokens
        assert list(r.output) == alone.generate([prompts[k]], [params[k]])[0], f"request {k}"


@pytest.mark.parametrize("lookahead", [False, True])
def test_preemption_by_recompute_in_bfloat16(lookahead):
    """Thirty greedy requests in bfloat16 through a cache that holds a fraction of them (head
    size 64: the fused decode kernel, recorded steps, the tcgen05 attention for the recomputed
    prompts).  Requests are preempted, lose their pages and are computed again from their
    prompt plus what they had generated; the plain implementation, reading each finished
    sequence, must agree with every token that was not a near-tie."""
    from llmario_b200 import Engine, SamplingParams
    name, dtype = "D", "bfloat16"
    rng = random.Random(6)
    prompts = [random_tokens(name, rng.randint(3, 90), 600 + i) for i in range(30)]
    params = [SamplingParams(temperature=0.0, max_tokens=rng.randint(8, 50)) for _ in range(30)]
    eng = Engine(model_dir(name, dtype), dtype=dtype, page_size=16, cache_tokens=352,
                 max_requests=6, context=256, token_budget=48, lookahead=lookahead)
    outs = eng.generate(prompts, params)
    cache = eng.runner.cache
    cache.check_invariants()
    assert min(cache.free_pages()) == cache.groups[0].n_pages and not cache.live_requests()
    st = eng.stats()
    assert st["preemptions"] > 0 and st["graph_replays"] > 0 and st["failed_steps"] == 0
    assert (st.get("steps_planned_ahead", 0) > 10) == lookahead
    assert [len(o) for o in outs] == [p.max_tokens for p in params]
    clear = sum(check_greedy_against_plain(name, dtype, p, o, f"request {i}")
                for i, (p, o) in enumerate(zip(prompts, outs)))
    assert clear >= 150


def test_patch_tokens_kernel():
    from llmario_b200 import kernels
    tokens = torch.arange(10, 20, dtype=torch.int32, device=DEV)
    source = torch.tensor([100, 200, 300], dtype=torch.int32, device=DEV)
    index = torch.tensor([-1, 2, 0, -1, 1, 1, -1, -1, 0, 2], dtype=torch.int32, device=DEV)
    kernels.patch_tokens(tokens, source, index)
    assert tokens.tolist() == [10, 300, 100, 13, 200, 200, 16, 17, 100, 300]


# ----------------------------------------------------------------------------- parts alone
def test_parts_alone():
    """Each part built from its spec and stepped by itself against the plain functions."""
    from llmario_b200.cache import CacheManager
    from llmario_b200.config import load_spec
    from llmario_b200.parts import BoundCall, Segment, StepContext, Workspace, build_part
    from llmario_b200.weights import load_weights
    name, dtype = "C", "float32"
    d = model_dir(name, dtype)
    spec = load_spec(d)
    weights = load_weights(d, spec, torch.float32, DEV)
    tensors, cfg = P.load(d)
    T, hidden = 23, spec.hidden_size
    x64 = torch.randn(T, hidden, dtype=torch.float64)
    x = x64.float().to(DEV)

    norm = build_part("norm", spec.final_norm, weights, torch.float32, DEV)
    out = torch.empty_like(x)
    norm.apply(None, x, out)
    ref = P.rms_norm(x64, tensors["model.norm.weight"], cfg["eps"])
    assert (out.double().cpu() - ref).abs().max() < 1e-5

    layer = spec.layers[1]                      # a layer with a window
    mixer = build_part("mixer", layer.mixer, weights, torch.float32, DEV)
    ffn = build_part("feed_forward", layer.feed_forward, weights, torch.float32, DEV)
    cache = CacheManager([mixer.cache_need()], [None], 16, 8, 2, 64)
    cache.allocate_storage(torch.float32, DEV)
    cache.open("r")
    cache.reserve([("r", T)])
    (upd,) = cache.take_table_updates()
    for s, j, p in upd:
        cache.groups[0].table[s, j] = int(p)
    ar = torch.arange(T, dtype=torch.int32, device=DEV)
    ctx = StepContext(rows=T, tokens=ar, row_pos=ar, row_slot=torch.zeros_like(ar),
                      segments=[Segment("r", 0, 0, T, 0)], dtype=torch.float32,
                      device=torch.device(DEV), workspace=Workspace(torch.device(DEV)), cache=cache)
    acc = torch.zeros_like(x)
    mixer.forward(ctx, BoundCall(0, 1, True, 0), x, acc)
    ref, _ = P.attention_mixer(x64, torch.arange(T), tensors, "model.layers.1.self_attn.", cfg,
                               cfg["windows"][1])
    assert cfg["windows"][1] == 21
    assert (acc.double().cpu() - ref).abs().max() < 1e-5

    acc.zero_()
    ffn.forward(ctx, x, acc)
    p = "model.layers.1.mlp."
    ref = P.swiglu_ffn(x64, tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"],
                       tensors[p + "down_proj.weight"])
    assert (acc.double().cpu() - ref).abs().max() < 1e-5

    emb = build_part("embedding", spec.embedding, weights, torch.float32, DEV)
    toks = torch.tensor(random_tokens(name, T, 1), dtype=torch.int32, device=DEV)
    e = torch.empty_like(x)
    emb.forward(ctx, toks, e)
    assert torch.equal(e.cpu(), tensors["model.embed_tokens.weight"][toks.cpu().long()].float())
    head = build_part("head", spec.head, weights, torch.float32, DEV)
    logits = torch.empty(T, spec.vocab_size, dtype=torch.float32, device=DEV)
    head.forward(ctx, x, logits)
    assert (logits.double().cpu() - P.linear(x64, tensors["lm_head.weight"])).abs().max() < 1e-4

    pos = build_part("position", layer.mixer["position"], weights, torch.float32, DEV)
    inv_freq, rot, factor = pos.rotary_tables()
    want = cfg["theta"] ** (-(2.0 * np.arange(rot // 2)) / rot)
    assert rot == cfg["head_dim"] and factor == 1.0
    assert np.abs(inv_freq.cpu().numpy() / want - 1).max() < 1e-6


# ----------------------------------------------------------------------------- a toy mixer
class RunningMeanMixer:
    """A mixer with a state of its own, defined here and not in the package: the state of a
    request is the running sum of its inputs and their count; the output at a token is
    W (mean of the inputs up to and including it)."""

    graph_safe = True     # a step of single tokens finds its state rows through ctx.row_slot

    def __init__(self, spec, weights, dtype, device):
        self.hidden = spec["hidden_size"]
        self.weight = weights[spec["tensors"]["mix"][0]].float()

    def cache_need(self):
        from llmario_b200.cache import FixedState
        return FixedState((self.hidden + 1,), torch.float32)

    def forward(self, ctx, call, h, x):
        state = ctx.cache.state_of(call.cache_entry)
        if all(seg.rows == 1 for seg in ctx.segments):
            # single tokens: everything through device tensors, so the step can be recorded
            slot = ctx.row_slot.long()
            s = state.index_select(0, slot)
            sums = s[:, :self.hidden] + h.float()
            counts = s[:, self.hidden] + 1
            x += (sums / counts[:, None]) @ self.weight.T
            state.index_copy_(0, slot, torch.cat([sums, counts[:, None]], 1))
            return
        for seg in ctx.segments:
            rows = h[seg.row_start:seg.row_start + seg.rows].float()
            s = state[seg.slot]
            sums = s[:self.hidden] + rows.cumsum(0)
            counts = s[self.hidden] + torch.arange(1, seg.rows + 1, device=h.device)
            x[seg.row_start:seg.row_start + seg.rows] += (sums / counts[:, None]) @ self.weight.T
            s[:self.hidden] = sums[-1]
            s[self.hidden] = counts[-1]


def toy_spec(spec):
    """Config A with the mixer of layer 1 replaced by the running-mean mixer."""
    from llmario_b200.config import PartSpec
    hidden = spec.hidden_size
    toy = PartSpec("running_mean", {"hidden_size": hidden,
                                    "tensors": {"mix": ("toy.mix.weight", (hidden, hidden))}})
    layers = list(spec.layers)
    layers[1] = dataclasses.replace(layers[1], mixer=toy)
    return dataclasses.replace(spec, layers=tuple(layers))


def test_a_toy_mixer_with_state_is_registered_built_and_stepped():
    from llmario_b200.config import load_spec
    from llmario_b200.engine import Model, ModelRunner, StepEntry
    from llmario_b200.parts import register_part, unregister_part
    from llmario_b200.weights import expected_tensors, random_tensors
    register_part("mixer", "running_mean", RunningMeanMixer, replace=True)
    try:
        spec = toy_spec(load_spec(model_dir("A", "float32")))
        names = expected_tensors(spec)
        assert "toy.mix.weight" in names and "model.layers.1.self_attn.q_proj.weight" not in names
        weights = random_tensors(spec, 5, torch.float32, DEV)
        host = {k: v.double().cpu() for k, v in weights.items()}
        model = Model(spec, weights, torch.float32, DEV)
        runner = ModelRunner(model, page_size=4, n_pages=32, max_requests=3, max_context=64)
        assert len(runner.cache.groups) == 1 and list(runner.cache.state) == [1]

        def reference(tokens):
            cfg = P.read_config(model_dir("A", "float32"))
            xx = P.embed(host["model.embed_tokens.weight"], tokens)
            pos = torch.arange(len(tokens))
            xx, _ = P.decoder_layer(xx, pos, host, 0, cfg)
            p = "model.layers.1."
            h = P.rms_norm(xx, host[p + "input_layernorm.weight"], cfg["eps"])
            mean = h.cumsum(0) / torch.arange(1, len(tokens) + 1)[:, None]
            xx = xx + mean @ host["toy.mix.weight"].T
            h = P.rms_norm(xx, host[p + "post_attention_layernorm.weight"], cfg["eps"])
            xx = xx + P.swiglu_ffn(h, host[p + "mlp.gate_proj.weight"], host[p + "mlp.up_proj.weight"],
                                   host[p + "mlp.down_proj.weight"])
            return P.linear(P.rms_norm(xx, host["model.norm.weight"], cfg["eps"]),
                            host["model.embed_tokens.weight"]).numpy()

        a, b = random_tokens("A", 21, 1), random_tokens("A", 13, 2)
        got = {"a": [], "b": []}
        # two requests interleaved in portions: each keeps a state of its own
        plan = [[("a", 0, 5)], [("a", 5, 3), ("b", 0, 6)], [("b", 6, 1)], [("a", 8, 13), ("b", 7, 6)]]
        toks = {"a": a, "b": b}
        for step in plan:
            entries = [StepEntry(r, toks[r][s:s + n], list(range(n))) for r, s, n in step]
            out = runner.step(entries).cpu().numpy()
            at = 0
            for r, s, n in step:
                got[r].append(out[at:at + n])
                at += n
        assert_close(np.concatenate(got["a"]), reference(a), "float32", "toy mixer a")
        assert_close(np.concatenate(got["b"]), reference(b), "float32", "toy mixer b")
        # steps of single tokens are recorded and replayed although the model keeps state;
        # a request that joins in the middle gets a fresh (zeroed) slot inside a replayed step
        assert model.graph_safe and runner.use_graphs
        more = {"a": random_tokens("A", 12, 3), "b": random_tokens("A", 12, 4)}
        c, d = random_tokens("A", 7, 5), random_tokens("A", 3, 6)
        tail = {"a": [], "b": [], "c": [], "d": []}
        for i in range(12):
            if i == 9:
                runner.close("c")      # d takes over c's slot, state and all, in a replayed step
            feed = {"a": more["a"][i], "b": more["b"][i]}
            if 2 <= i < 9:
                feed["c"] = c[i - 2]
            if i >= 9:
                feed["d"] = d[i - 9]
            out = runner.step([StepEntry(r, [t], [0]) for r, t in feed.items()]).cpu().numpy()
            for j, r in enumerate(feed):
                tail[r].append(out[j:j + 1])
        assert runner.counters["graph_replays"] >= 6
        assert runner.cache.slot("d") is not None
        assert_close(np.concatenate(tail["a"]), reference(a + more["a"])[len(a):], "float32",
                     "toy mixer a, recorded steps")
        assert_close(np.concatenate(tail["b"]), reference(b + more["b"])[len(b):], "float32",
                     "toy mixer b, recorded steps")
        assert_close(np.concatenate(tail["c"]), reference(c), "float32",
                     "toy mixer c, joined a recorded step")
        assert_close(np.concatenate(tail["d"]), reference(d), "float32",
                     "toy mixer d, a used slot zeroed inside a replayed step")
        # a slot that is used again starts from a zero state
        runner.close("a"), runner.close("b"), runner.close("d")
        out = runner.step([StepEntry("c", b, list(range(len(b))))]).cpu().numpy()
        assert_close(out, reference(b), "float32", "toy mixer, slot used again")
    finally:
        unregister_part("mixer", "running_mean")


class TwoMixerBlock:
    """A block defined here with two stateful mixers, each with a cache entry of its own:
    ``x += first(norm(x)); x += second(norm(x)); x += feed_forward(norm(x))``."""

    def __init__(self, spec, layer, weights, dtype, device):
        from llmario_b200.parts import build_part
        self.norm = build_part("norm", spec["norm"], weights, dtype, device)
        self.ffn_norm = build_part("norm", spec["feed_forward_norm"], weights, dtype, device)
        self.first = build_part("mixer", layer.mixer, weights, dtype, device)
        self.second = build_part("mixer", spec["second_mixer"], weights, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, dtype, device)
        self.graph_safe = True

    def cache_needs(self):
        return [self.first.cache_need(), self.second.cache_need()]

    def forward(self, ctx, call, x):
        h = ctx.buffer("block.h", x.shape)
        self.norm.apply(ctx, x, h)
        self.first.forward(ctx, call.for_need(0), h, x)
        self.norm.apply(ctx, x, h)
        self.second.forward(ctx, call.for_need(1), h, x)
        self.ffn_norm.apply(ctx, x, h)
        self.feed_forward.forward(ctx, h, x)


def test_a_toy_block_with_two_stateful_mixers():
    """Registered, built and stepped from here; ``engine/`` is untouched.  Every need of the
    block gets its own state tensor, and the steps of single tokens are replayed as graphs."""
    from llmario_b200.config import PartSpec, load_spec
    from llmario_b200.engine import Model, ModelRunner, StepEntry
    from llmario_b200.parts import register_part, unregister_part
    from llmario_b200.weights import random_tensors
    register_part("mixer", "running_mean", RunningMeanMixer, replace=True)
    register_part("block", "two_mixers", TwoMixerBlock, replace=True)
    try:
        spec = load_spec(model_dir("A", "float32"))
        hidden = spec.hidden_size
        mixers = [PartSpec("running_mean", {"hidden_size": hidden, "tensors": {
            "mix": (f"toy.mix{k}.weight", (hidden, hidden))}}) for k in (0, 1)]
        old = spec.layers[1]
        block = PartSpec("two_mixers", {"norm": old.block["mixer_norm"],
                                        "feed_forward_norm": old.block["feed_forward_norm"],
                                        "second_mixer": mixers[1]})
        layers = (spec.layers[0], dataclasses.replace(old, block=block, mixer=mixers[0]))
        spec = dataclasses.replace(spec, layers=layers)
        weights = random_tensors(spec, 6, torch.float32, DEV)
        assert "toy.mix0.weight" in weights and "toy.mix1.weight" in weights
        host = {k: v.double().cpu() for k, v in weights.items()}
        model = Model(spec, weights, torch.float32, DEV)
        assert model.calls[1].cache_entries == (1, 2) and model.calls[0].cache_entries == (0,)
        runner = ModelRunner(model, page_size=4, n_pages=32, max_requests=3, max_context=64)
        assert sorted(runner.cache.state) == [1, 2] and runner.use_graphs

        def reference(tokens):
            cfg = P.read_config(model_dir("A", "float32"))
            xx = P.embed(host["model.embed_tokens.weight"], tokens)
            xx, _ = P.decoder_layer(xx, torch.arange(len(tokens)), host, 0, cfg)
            p = "model.layers.1."
            for k in (0, 1):
                h = P.rms_norm(xx, host[p + "input_layernorm.weight"], cfg["eps"])
                mean = h.cumsum(0) / torch.arange(1, len(tokens) + 1)[:, None]
                xx = xx + mean @ host[f"toy.mix{k}.weight"].T
            h = P.rms_norm(xx, host[p + "post_attention_layernorm.weight"], cfg["eps"])
            xx = xx + P.swiglu_ffn(h, host[p + "mlp.gate_proj.weight"], host[p + "mlp.up_proj.weight"],
                                   host[p + "mlp.down_proj.weight"])
            return P.linear(P.rms_norm(xx, host["model.norm.weight"], cfg["eps"]),
                            host["model.embed_tokens.weight"]).numpy()

        a, b = random_tokens("A", 17, 7), random_tokens("A", 12, 8)
        got = {"a": [runner.step([StepEntry("a", a[:6], list(range(6)))]).cpu().numpy()], "b": []}
        out = runner.step([StepEntry("a", a[6:9], [0, 1, 2]), StepEntry("b", b[:4], [0, 1, 2, 3])])
        got["a"].append(out[:3].cpu().numpy()), got["b"].append(out[3:].cpu().numpy())
        for i in range(8):
            out = runner.step([StepEntry("a", [a[9 + i]], [0]), StepEntry("b", [b[4 + i]], [0])])
            got["a"].append(out[:1].cpu().numpy()), got["b"].append(out[1:].cpu().numpy())
        assert runner.counters["graph_replays"] >= 5
        assert_close(np.concatenate(got["a"]), reference(a), "float32", "two mixers a")
        assert_close(np.concatenate(got["b"]), reference(b), "float32", "two mixers b")
    finally:
        unregister_part("mixer", "running_mean")
        unregister_part("block", "two_mixers")


# ------------------------------------------------- a toy feed-forward and a toy position encoding
class TopOneOfTwo:
    """A feed-forward with routing, defined here and not in the package: a router scores two
    small gated experts per token in 32-bit, the token goes to the better one and the expert's
    output is weighted by the softmax probability of its score."""

    def __init__(self, spec, weights, dtype, device):
        t = spec["tensors"]
        self.router = weights[t["router"][0]].float()
        self.experts = [tuple(weights[t[f"{r}{e}"][0]].float() for r in ("gate", "up", "down"))
                        for e in range(2)]

    def forward(self, ctx, h, x):
        hf = h.float()
        scores = hf @ self.router.T
        prob = torch.softmax(scores, -1)
        choice = scores.argmax(-1)
        for e, (gate, up, down) in enumerate(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                g = hf[rows] @ gate.T
                y = (g / (1 + torch.exp(-g)) * (hf[rows] @ up.T)) @ down.T
                x.index_add_(0, rows, y * prob[rows, e:e + 1])


class InterpolatedPartialRotary:
    """A position encoding defined here: only the first half of each head is rotated, positions
    are divided by a factor (interpolation), and the rotated values are scaled by a constant.
    It offers no per-step table, so the fused kernel computes the angles itself."""

    def __init__(self, spec, weights, dtype, device):
        self.rot_dim, self.theta = int(spec["rot_dim"]), float(spec["theta"])
        self.factor, self.gain = float(spec["factor"]), float(spec["gain"])
        i = np.arange(self.rot_dim // 2, dtype=np.float64)
        freq = self.theta ** (-(2.0 * i) / self.rot_dim) / self.factor
        self.inv_freq = torch.tensor(freq.astype(np.float32), device=device)

    def rotary_tables(self):
        return self.inv_freq, self.rot_dim, self.gain


def test_a_toy_feed_forward_with_routing_and_a_toy_position_encoding():
    """Both are registered from here, chosen by a spec for layer 1 of config A, built and
    stepped in portions and in a mixed batch; the framework's files are untouched."""
    from llmario_b200.config import PartSpec, load_spec
    from llmario_b200.engine import Model, ModelRunner, StepEntry
    from llmario_b200.parts import register_part, unregister_part
    from llmario_b200.weights import expected_tensors, random_tensors
    register_part("feed_forward", "top_one_of_two", TopOneOfTwo, replace=True)
    register_part("position", "interpolated_partial", InterpolatedPartialRotary, replace=True)
    try:
        base = load_spec(model_dir("A", "float32"))
        cfg = P.read_config(model_dir("A", "float32"))
        hidden, ff, hd = base.hidden_size, 24, cfg["head_dim"]
        tensors = {"router": ("toy.router.weight", (2, hidden))}
        for e in range(2):
            tensors[f"gate{e}"] = (f"toy.expert{e}.gate.weight", (ff, hidden))
            tensors[f"up{e}"] = (f"toy.expert{e}.up.weight", (ff, hidden))
            tensors[f"down{e}"] = (f"toy.expert{e}.down.weight", (hidden, ff))
        routed = PartSpec("top_one_of_two", {"hidden_size": hidden, "tensors": tensors})
        rot, factor, gain = hd // 2, 4.0, 1.25
        position = PartSpec("interpolated_partial", {"rot_dim": rot, "theta": 5000.0,
                                                     "factor": factor, "gain": gain})
        layers = list(base.layers)
        mixer = dataclasses.replace(layers[1].mixer,
                                    params={**layers[1].mixer.params, "position": position})
        layers[1] = dataclasses.replace(layers[1], mixer=mixer, feed_forward=routed)
        spec = dataclasses.replace(base, layers=tuple(layers))
        names = expected_tensors(spec)
        assert "toy.router.weight" in names and "model.layers.1.mlp.up_proj.weight" not in names
        weights = random_tensors(spec, 11, torch.float32, DEV)
        host = {k: v.double().cpu() for k, v in weights.items()}
        runner = ModelRunner(Model(spec, weights, torch.float32, DEV), page_size=4, n_pages=40,
                             max_requests=3, max_context=64)

        def rotate(x, positions, heads):      # first `rot` dims of each head, pairs (i, i + rot/2)
            t = x.shape[0]
            xh = x.reshape(t, heads, hd).clone()
            i = torch.arange(rot // 2, dtype=torch.float64)
            freq = torch.tensor(5000.0, dtype=torch.float64) ** (-(2.0 * i) / rot) / factor
            ang = positions.double()[:, None] * freq[None, :]
            cos, sin = torch.cos(ang)[:, None, :] * gain, torch.sin(ang)[:, None, :] * gain
            a, b = xh[..., :rot // 2].clone(), xh[..., rot // 2:rot].clone()
            xh[..., :rot // 2] = a * cos - b * sin
            xh[..., rot // 2:rot] = a * sin + b * cos
            return xh.reshape(t, heads * hd)

        def reference(tokens):
            xx = P.embed(host["model.embed_tokens.weight"], tokens)
            pos = torch.arange(len(tokens))
            xx, _ = P.decoder_layer(xx, pos, host, 0, cfg)
            p = "model.layers.1."
            h = P.rms_norm(xx, host[p + "input_layernorm.weight"], cfg["eps"])
            hq, hkv = cfg["heads"], cfg["kv_heads"]
            q = P.per_head_norm(P.linear(h, host[p + "self_attn.q_proj.weight"]),
                                host[p + "self_attn.q_norm.weight"], cfg["eps"], hq)
            k = P.per_head_norm(P.linear(h, host[p + "self_attn.k_proj.weight"]),
                                host[p + "self_attn.k_norm.weight"], cfg["eps"], hkv)
            v = P.linear(h, host[p + "self_attn.v_proj.weight"])
            a = P.attention(rotate(q, pos, hq), rotate(k, pos, hkv), v, hq, hkv, hd,
                            cfg["windows"][1], pos)
            xx = xx + P.linear(a, host[p + "self_attn.o_proj.weight"])
            h = P.rms_norm(xx, host[p + "post_attention_layernorm.weight"], cfg["eps"])
            scores = h @ host["toy.router.weight"].T
            prob = torch.softmax(scores, -1)
            y = torch.zeros_like(xx)
            for t in range(len(tokens)):
                e = int(scores[t].argmax())
                g = h[t] @ host[f"toy.expert{e}.gate.weight"].T
                u = h[t] @ host[f"toy.expert{e}.up.weight"].T
                y[t] = ((g / (1 + torch.exp(-g)) * u) @ host[f"toy.expert{e}.down.weight"].T) * prob[t, e]
            xx = xx + y
            return P.linear(P.rms_norm(xx, host["model.norm.weight"], cfg["eps"]),
                            host["model.embed_tokens.weight"]).numpy()

        a, b = random_tokens("A", 23, 3), random_tokens("A", 9, 4)
        toks, got = {"a": a, "b": b}, {"a": [], "b": []}
        plan = [[("a", 0, 7)], [("a", 7, 2), ("b", 0, 8)], [("a", 9, 1), ("b", 8, 1)], [("a", 10, 13)]]
        for step in plan:
            entries = [StepEntry(r, toks[r][s:s + n], list(range(n))) for r, s, n in step]
            out = runner.step(entries).cpu().numpy()
            at = 0
            for r, s, n in step:
                got[r].append(out[at:at + n])
                at += n
        ref_a, ref_b = reference(a), reference(b)
        assert_close(np.concatenate(got["a"]), ref_a, "float32", "toy routed feed-forward a")
        assert_close(np.concatenate(got["b"]), ref_b, "float32", "toy routed feed-forward b")
    finally:
        unregister_part("feed_forward", "top_one_of_two")
        unregister_part("position", "interpolated_partial")


# ------------------------------------------- options of the standard parts this architecture leaves off
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_projection_biases_and_adjacent_pair_rotation(dtype):
    """Two options that the standard parts take as data although this architecture uses
    neither: biases of the q, k, v and output projections (added after the product,
    forward.rs:399-425) and the rotation of adjacent pairs (2i, 2i+1) (``RopeKind::Normal``,
    ops.rs:57-60), here on part of a head, with scaled positions and a factor on cosine and
    sine.  Layer 0 has the other rotation only and runs through the native step driver; layer
    1 has both and runs through the parts' own forward.  Compared with the formulas in float64,
    in portions, in a mixed step and token by token."""
    from llmario_b200.config import PartSpec, load_spec
    from llmario_b200.engine import Model, ModelRunner, StepEntry
    from llmario_b200.weights import expected_tensors, random_tensors

    name = "D"
    base = load_spec(model_dir(name, dtype))
    cfg = P.read_config(model_dir(name, dtype))
    hq, hkv, hd, eps = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["eps"]
    rotation = [dict(rot_dim=hd, theta=cfg["theta"], freq_scale=1.0, attn_factor=1.0),
                dict(rot_dim=hd // 2, theta=3000.0, freq_scale=0.5, attn_factor=1.125)]
    layers = list(base.layers)
    for l in range(2):
        params = dict(layers[l].mixer.params)
        params["position"] = PartSpec("rope_normal", rotation[l])
        if l == 1:
            a = "model.layers.1.self_attn."
            tensors = dict(params["tensors"])
            for r, width in (("q", hq * hd), ("k", hkv * hd), ("v", hkv * hd), ("o", base.hidden_size)):
                tensors[r + "_bias"] = (a + r + "_proj.bias", (width,))
            params["tensors"] = tensors
        layers[l] = dataclasses.replace(layers[l], mixer=dataclasses.replace(layers[l].mixer,
                                                                             params=params))
    spec = dataclasses.replace(base, layers=tuple(layers))
    assert "model.layers.1.self_attn.k_proj.bias" in expected_tensors(spec)
    tdtype = getattr(torch, dtype)
    weights = random_tensors(spec, 21, tdtype, DEV)
    gen = torch.Generator().manual_seed(5)
    for n in list(weights):
        if n.endswith(".bias"):      # (the seeded generator makes gains near one for 1-D tensors)
            weights[n] = (0.4 * torch.randn(weights[n].shape, generator=gen)).to(DEV)
    host = {k: v.double().cpu() for k, v in weights.items()}
    runner = ModelRunner(Model(spec, weights, tdtype, DEV), page_size=16, n_pages=24,
                         max_requests=3, max_context=128)
    assert runner.native is not None and runner.native.native_layer == [True, False]

    def reference(tokens):
        xx = P.embed(host["model.embed_tokens.weight"], tokens)
        pos = torch.arange(len(tokens))
        for l in range(2):
            p = f"model.layers.{l}."
            a, rot = p + "self_attn.", rotation[l]
            h = P.rms_norm(xx, host[p + "input_layernorm.weight"], eps)
            proj = {r: P.linear(h, host[a + r + "_proj.weight"], host.get(a + r + "_proj.bias"))
                    for r in ("q", "k", "v")}
            q = P.per_head_norm(proj["q"], host[a + "q_norm.weight"], eps, hq)
            k = P.per_head_norm(proj["k"], host[a + "k_norm.weight"], eps, hkv)
            turn = lambda t, heads: P.rope_normal(t, pos, heads, hd, rot["rot_dim"], rot["theta"],
                                                  rot["freq_scale"], rot["attn_factor"])
            att = P.attention(turn(q, hq), turn(k, hkv), proj["v"], hq, hkv, hd,
                              cfg["windows"][l], pos)
            xx = xx + P.linear(att, host[a + "o_proj.weight"], host.get(a + "o_proj.bias"))
            h = P.rms_norm(xx, host[p + "post_attention_layernorm.weight"], eps)
            xx = xx + P.swiglu_ffn(h, host[p + "mlp.gate_proj.weight"],
                                   host[p + "mlp.up_proj.weight"], host[p + "mlp.down_proj.weight"])
        return P.linear(P.rms_norm(xx, host["model.norm.weight"], eps),
                        host["lm_head.weight"]).numpy()

    a, b = random_tokens(name, 45, 31), random_tokens(name, 27, 32)
    toks, got = {"a": a, "b": b}, {"a": [], "b": []}
    plan = [[("a", 0, 19)], [("a", 19, 14), ("b", 0, 17)], [("a", 33, 2), ("b", 17, 1)]]
    plan += [[("a", 35 + i, 1), ("b", 18 + i, 1)] for i in range(9)]       # recorded decode steps
    plan += [[("a", 44, 1)]]
    for step in plan:
        entries = [StepEntry(r, toks[r][s:s + n], list(range(n))) for r, s, n in step]
        out = runner.step(entries).cpu().numpy()
        at = 0
        for r, s, n in step:
            got[r].append(out[at:at + n])
            at += n
    assert runner.counters["graph_replays"] >= 5
    assert_close(np.concatenate(got["a"]), reference(a), dtype, "biases, adjacent pairs a", name)
    assert_close(np.concatenate(got["b"]), reference(b), dtype, "biases, adjacent pairs b", name)
