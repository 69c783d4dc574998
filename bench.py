#!/usr/bin/env python3
"""Decode and prefill rates of the engine on one B200, as one JSON line.

    python bench.py --gpus 1 --steps K --warmup W [--model NAME] [--workload decode|serve]

``--workload decode`` (the default).  A "step" is one decode step of a batch of requests.  The
default run has the layer sizes of Qwen3-8B with seeded random bfloat16 weights, 8 requests with
1,024-token prompts of uniform random ids, context 8,192, pages of 16 tokens (the named
configuration).  ``value`` is decoded tokens per second timed on the device around K consecutive
steps of the step function plus the sampling kernel; ``e2e`` is the same through ``Engine.step``
with host token lists in and out (prompts run as steps of thousands of tokens at the power cap
and the SM clock stays low for some 60 ms after them, so at least 48 untimed decode steps,
``config.untimed_steps``, come before the K timed ones, of both figures); ``prefill`` is one prompt of 2,048 tokens (median of the runs,
all runs listed); ``points`` holds batch 1 and 64; ``engine_page`` repeats prefill, ``value`` and
``e2e`` with the engine's default page of 64 tokens.  ``--model qwen3-32b --prompt-len 4096
--context 16384`` is the second named configuration.  The weights are larger than the L2 cache,
so no flush is needed between steps.

``--workload serve``.  The named workload of the small configuration (``--model qwen3-0.6b``):
32 requests arrive at once with prompt lengths uniform in [16, 2048] (seeded) and 128 decoded
tokens each, and run through ``Engine.add_request`` / ``Engine.step``: continuous batching with
prompts cut into portions under the token budget.  A "step" is then one engine step; ``value``
is generated tokens per second over the whole run (median of K runs after W warm-up runs), with
the reference's per-request figures (docs/BENCHMARK_PLAN.md:28-42: prefill = prompt tokens /
time to first token, decode = (completion - 1) / (t_last - t_first)), the fraction of the memory
roofline that the decode-only steps reach, and the host's share of the mixed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NAMES = {"qwen3-8b": "Qwen3-8B", "qwen3-0.6b": "Qwen3-0.6B", "qwen3-32b": "Qwen3-32B",
         "tiny-a": "tiny A", "tiny-b": "tiny B"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def summary(self, first: int = 0, last=None):
        """Median SM clock and the reasons seen in the samples [first, last)."""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines[first:last]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()


def reference_arm():
    """The reference is a Rust workspace (no Python package, no setup.py / pyproject.toml) and
    there is no Rust toolchain in the image, so it cannot be installed or run here."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "mannysinghx/LLMario is a Rust workspace without a Python package: pip "
                      "cannot install it, no cargo/rustc offline, and it has no CUDA backend"}))
    return 0


# Untimed decode steps between the prompts and the timed steps, at least: prompts run as steps of
# thousands of tokens at the power cap, and the SM clock stays low for some 60 ms after them
# (1,620 of 1,965 MHz; a decode step of Qwen3-8B sizes then takes 3.46 instead of 3.14 ms).  The
# timed steps start when that has passed, whatever --warmup says beyond it.
SETTLE_STEPS = 48


def decode_bench(runner, model, batch, prompt_len, steps, warmup, rng, chunk=2048):
    """Prefill ``batch`` requests of ``prompt_len`` tokens, then time ``steps`` decode steps on
    the device.  Returns (ms per step, cache bytes read per step on average, launches)."""
    import torch

    from llmario_b200 import kernels
    from llmario_b200.benchmarks.roofline import kv_bytes_per_token
    from llmario_b200.engine import StepEntry

    vocab = model.vocab_size
    warmup = max(warmup, SETTLE_STEPS)
    ids = [f"b{batch}-{i}" for i in range(batch)]
    for rid in ids:
        toks = [rng.randrange(vocab) for _ in range(prompt_len)]
        for at in range(0, prompt_len, chunk):
            runner.step([StepEntry(rid, toks[at:at + chunk], [])])
    feed = [[rng.randrange(vocab) for _ in ids] for _ in range(warmup + steps)]
    dev = model.device
    bufs = {"t": torch.zeros(batch, device=dev), "k": torch.zeros(batch, dtype=torch.int32, device=dev),
            "p": torch.ones(batch, device=dev), "m": torch.zeros(batch, device=dev),
            "u": torch.zeros(batch, dtype=torch.float64, device=dev),
            "o": torch.zeros(batch, dtype=torch.int32, device=dev)}

    def one(i):
        logits = runner.step([StepEntry(rid, [feed[i][j]], [0]) for j, rid in enumerate(ids)])
        kernels.sample(logits, bufs["t"], bufs["k"], bufs["p"], bufs["m"], bufs["u"], bufs["o"])

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    l0 = kernels.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = kernels.launches - l0
    mean_len = prompt_len + warmup + (steps - 1) / 2.0 + 1
    kv_bytes = batch * mean_len * kv_bytes_per_token(runner)
    for rid in ids:
        runner.close(rid)
    return ms, kv_bytes, launches


def e2e_bench(engine, batch, prompt_len, steps, warmup, rng):
    """The same decode steps through Engine.step: host token lists in, host token ids out."""
    import torch

    from llmario_b200.sampling import SamplingParams

    vocab = engine.model.vocab_size
    # (no request may end inside the timed region: the first ones to finish their prompts decode
    # while the others are still being prefilled, so they are ahead by a few tokens)
    params = SamplingParams(temperature=0.0, max_tokens=1 << 30, ignore_eos=True)
    ids = [engine.add_request([rng.randrange(vocab) for _ in range(prompt_len)], params)
           for _ in range(batch)]
    while not all(engine.request(i).output for i in ids):
        engine.step()                      # prefill (chunked under the token budget)
    # (the untimed steps go on until the clocks have recovered from the prompts: SETTLE_STEPS)
    for _ in range(max(warmup, SETTLE_STEPS)):
        engine.step()
    torch.cuda.synchronize()
    st0 = engine.stats()
    t0 = time.perf_counter()
    n0 = sum(len(engine.request(i).output) for i in ids)
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    st1 = engine.stats()
    n1 = sum(len(engine.request(i).output) for i in ids)
    for i in ids:
        engine.abort(i)
    # bytes the engine copied to and from the device per step, counted where it copies them
    copied = ((st1["h2d_bytes"] - st0["h2d_bytes"]) / steps, (st1["d2h_bytes"] - st0["d2h_bytes"]) / steps)
    return (n1 - n0) / (t1 - t0), copied


def prefill_bench(runner, model, tokens, rng, reps=5):
    """One prompt of ``tokens`` tokens in one step, logits at its last place: the times of
    ``reps`` runs in ms (after one untimed run)."""
    import torch

    from llmario_b200.engine import StepEntry

    vocab = model.vocab_size
    times = []
    for r in range(reps + 1):
        toks = [rng.randrange(vocab) for _ in range(tokens)]
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(f"p{r}", toks, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.close(f"p{r}")
        if r > 0:
            times.append(start.elapsed_time(end))
    return times


def prefill_record(model, times_ms, tokens, pk):
    from llmario_b200.benchmarks.roofline import prefill_flops

    ms = statistics.median(times_ms)
    flops = prefill_flops(model, tokens)
    rate = flops / (ms / 1e3)
    # frac: against the burst peak (a prompt is a short, isolated piece of work here); the
    # sustained peak is what a long run under the power cap reaches
    return {"value": tokens / (ms / 1e3), "tokens": tokens, "ms": ms,
            "frac": rate / (pk["bf16_tflops"] * 1e12),
            "frac_sustained": rate / (pk["bf16_tflops_sustained"] * 1e12),
            "tflops": rate / 1e12, "runs_ms": [round(t, 3) for t in times_ms],
            "best_ms": min(times_ms)}


def serve_workload(args, cfg, model, pk, clocks):
    """32 requests (``--requests``) with prompt lengths uniform in [16, 2048] and 128 decoded
    tokens each through the engine's own loop."""
    import torch

    from llmario_b200 import kernels
    from llmario_b200.benchmarks.roofline import kv_bytes_per_token
    from llmario_b200.engine.engine import Engine
    from llmario_b200.sampling import SamplingParams

    n, new = args.requests, args.decode_len
    rng = random.Random(args.seed)
    lengths = [rng.randint(args.min_prompt, args.max_prompt) for _ in range(n)]
    page = args.page_size
    cache_tokens = sum(-(-(l + new + 1) // page) * page for l in lengths) + 4 * page
    slots = min(n, args.max_requests or n)
    engine = Engine(model, page_size=page, cache_tokens=cache_tokens,
                    token_budget=args.token_budget, max_requests=slots, context=args.context)
    vocab = model.vocab_size
    weight_bytes = model.weight_bytes()
    kv_tok = kv_bytes_per_token(engine.runner)
    real_step = engine.runner.step
    host = {"mixed_s": 0.0, "mixed_steps": 0, "decode_s": 0.0, "decode_steps": 0}
    log = []                          # per launched step: (decode only?, bytes it has to read)

    def timed_step(entries, device_tokens=None):
        t0 = time.perf_counter()
        out = real_step(entries, device_tokens)
        dt = time.perf_counter() - t0
        only = all(len(e.tokens) == 1 for e in entries)
        ctx_tokens = sum(engine.runner.length(e.request) for e in entries)   # after the step
        log.append((only, weight_bytes + ctx_tokens * kv_tok))
        host["decode_s" if only else "mixed_s"] += dt
        host["decode_steps" if only else "mixed_steps"] += 1
        return out

    engine.runner.step = timed_step
    runs = []
    first_mark = None
    for it in range(args.warmup + args.steps):
        for k in host:
            host[k] = 0
        log.clear()
        prompts = [[rng.randrange(vocab) for _ in range(l)] for l in lengths]
        params = SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True)
        torch.cuda.synchronize()
        if it == args.warmup:
            first_mark = clocks.mark()
        l0 = kernels.launches
        st0 = engine.stats()
        t0 = time.perf_counter()
        ids = [engine.add_request(p, params) for p in prompts]
        t_first, t_last = {}, {}
        waiting = set(ids)
        stamps = []                  # completion time of every engine step
        while engine.has_work():
            done = engine.step()
            now = time.perf_counter()
            stamps.append(now)
            for rid in list(waiting):
                if engine.request(rid).output:
                    t_first[rid] = now
                    waiting.discard(rid)
            for r in done:
                t_last[r.id] = now
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        gen = sum(len(engine.request(i).output) for i in ids)
        assert gen == n * new and all(engine.request(i).finish_reason == "length" for i in ids)
        # decode-only steps: the stretch after the last mixed step, by completion stamps (with a
        # step queued ahead the stamps follow the device, one step apart)
        last_mixed = max((i for i, (only, _) in enumerate(log) if not only), default=-1)
        tail = [b for only, b in log[last_mixed + 1:]]
        roof = None
        k = min(len(tail), len(stamps) - 1)
        if k > 8:
            span = stamps[-1] - stamps[-1 - (k - 4)]
            gbs = sum(tail[-(k - 4):]) / span / 1e9
            roof = {"steps": k - 4, "achieved": gbs, "frac": gbs / pk["hbm_gbs"],
                    "ms_per_step": span / (k - 4) * 1e3}
        per_req_decode = [(new - 1) / max(t_last[i] - t_first[i], 1e-9) for i in ids]
        per_req_prefill = [l / (t_first[i] - t0) for i, l in zip(ids, lengths)]
        if it >= args.warmup:
            runs.append({
                "seconds": t1 - t0, "aggregate_tok_s": gen / (t1 - t0),
                "total_tok_s": (gen + sum(lengths)) / (t1 - t0),
                "decode_tok_s_per_request": statistics.median(per_req_decode),
                "prefill_tok_s_per_request": statistics.median(per_req_prefill),
                "ttft_ms_median": statistics.median((t_first[i] - t0) * 1e3 for i in ids),
                "ttft_ms_max": max((t_first[i] - t0) * 1e3 for i in ids),
                "engine_steps": len(stamps), "mixed_steps": host["mixed_steps"],
                "steps_queued_ahead": engine.stats()["steps_planned_ahead"] - st0["steps_planned_ahead"],
                "request_slots": slots,
                "host_ms_per_mixed_step": host["mixed_s"] / max(1, host["mixed_steps"]) * 1e3,
                "host_ms_per_decode_step": host["decode_s"] / max(1, host["decode_steps"]) * 1e3,
                "mixed_wall_s": (stamps[last_mixed] - t0) if last_mixed >= 0 else 0.0,
                "host_share_of_mixed": host["mixed_s"] / max(1e-9, (stamps[last_mixed] - t0))
                if last_mixed >= 0 else None,
                "decode_roofline": roof, "launches": kernels.launches - l0,
                "h2d_bytes_per_step": (engine.stats()["h2d_bytes"] - st0["h2d_bytes"]) / len(stamps),
                "d2h_bytes_per_step": (engine.stats()["d2h_bytes"] - st0["d2h_bytes"]) / len(stamps)})
        for i in ids:
            engine.release(i)
    clk = clocks.summary(first_mark)
    best = sorted(runs, key=lambda r: r["aggregate_tok_s"])[len(runs) // 2]
    name = NAMES.get(args.model, args.model)
    roof = best["decode_roofline"] or {"achieved": 0.0, "frac": 0.0}
    line = {
        "metric": f"generated tok/s of {n} concurrent requests, prompts U[{args.min_prompt}, "
                  f"{args.max_prompt}], {new} decoded each, continuous batching ({name} sizes, "
                  "random bf16 weights)",
        "value": best["aggregate_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": best["seconds"] * 1e3 / best["engine_steps"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, seeded prompt lengths, seeded random "
                "weights", "impl": "ours", "workload": "serve",
        "config": {"model": args.model, "layers": cfg.num_hidden_layers,
                   "layers_full": cfg.num_hidden_layers if not args.layers else
                   _full_layers(args.model), "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
                   "vocab": cfg.vocab_size, "global_batch": n, "seq_len": args.max_prompt,
                   "decode_len": new, "context": args.context, "page_size": page,
                   "token_budget": args.token_budget, "parallelism": "single GPU",
                   "l2": "every step reads the weights (%.2f GB), larger than L2" %
                         (weight_bytes / 1e9), "peaks": pk["source"]},
        "e2e": {"value": best["aggregate_tok_s"], "unit": "tokens/s",
                "note": "the whole workload runs through Engine.add_request / Engine.step: host "
                        "token lists in, host token ids out",
                "h2d_bytes_per_step": best["h2d_bytes_per_step"],
                "d2h_bytes_per_step": best["d2h_bytes_per_step"]},
        "gpu_launches": best["launches"], "clocks": clk, "runs": runs,
        "roofline": {"bound": "hbm", "achieved": roof["achieved"], "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": roof["frac"],
                     "of": "the decode-only steps at the end of the run"},
        "prompt_tokens": sum(lengths),
    }
    print(json.dumps(line))
    return 0


def _full_layers(model: str) -> int:
    from llmario_b200.cli import PRESETS

    return PRESETS[model]["num_hidden_layers"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="decode: timed steps (default 128); serve: timed runs (default 3)")
    ap.add_argument("--warmup", type=int, default=None,
                    help="decode: warm-up steps (default 8, at least 3); serve: warm-up runs "
                         "(default 1)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve"])
    ap.add_argument("--layers", type=int, default=None, help="build fewer layers (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--context", type=int, default=None,
                    help="per-request context (default 8192; serve: 4096)")
    ap.add_argument("--page-size", type=int, default=16,
                    help="tokens in a cache page for the headline numbers (the named configuration "
                         "has 16; the engine's own default, 64, is measured too and reported "
                         "under `engine_page`)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    # the serve workload
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--max-requests", type=int, default=None,
                    help="serve: request slots of the engine (default: all requests at once); "
                         "fewer make the rest wait for a slot")
    ap.add_argument("--min-prompt", type=int, default=16)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--decode-len", type=int, default=128)
    ap.add_argument("--token-budget", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    import torch

    from llmario_b200.benchmarks.roofline import peaks
    from llmario_b200.cli import preset_config
    from llmario_b200.engine import Model
    from llmario_b200.engine.engine import Engine

    pk = peaks()
    cfg = preset_config(args.model, args.layers)
    full_layers = _full_layers(args.model)
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    clocks = ClockSampler()
    clocks.start()
    try:
        if args.workload == "serve":
            args.steps = 3 if args.steps is None else args.steps
            args.warmup = 1 if args.warmup is None else args.warmup
            args.context = args.context or 4096
            return serve_workload(args, cfg, model, pk, clocks)
        return decode_workload(args, cfg, full_layers, model, pk, clocks)
    finally:
        clocks.stop()


def decode_workload(args, cfg, full_layers, model, pk, clocks):
    import torch

    from llmario_b200.engine.engine import Engine

    steps = 128 if args.steps is None else args.steps
    warmup = max(3, 8 if args.warmup is None else args.warmup)
    context = args.context or 8192
    rng = random.Random(0)
    max_batch = args.batch if args.skip_points else max(args.batch, 64)
    budget = max(2048, args.prefill_tokens)
    # room for the prompt, the decoded tokens and the tokens a request decodes while the prompts
    # of the others are still being prefilled
    ahead = args.batch * -(-args.prompt_len // budget) + 2
    per_req = args.prompt_len + max(warmup, SETTLE_STEPS) + steps + ahead + args.page_size
    cache_tokens = max(max_batch * per_req, args.prefill_tokens + args.page_size)
    engine = Engine(model, page_size=args.page_size, cache_tokens=cache_tokens,
                    token_budget=budget, max_requests=max_batch, context=context)
    runner = engine.runner
    weight_bytes = model.weight_bytes()
    c = cfg
    T = args.prefill_tokens

    # prefill first: it also warms every kernel
    prefill = prefill_record(model, prefill_bench(runner, model, T, rng), T, pk)
    mark = clocks.mark()
    ms, kv_bytes, launches = decode_bench(runner, model, args.batch, args.prompt_len, steps,
                                          warmup, rng)
    clk = clocks.summary(mark)
    value = args.batch / (ms / 1e3)
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9
    e2e, copied = e2e_bench(engine, args.batch, args.prompt_len, steps, warmup, rng)
    points = {}
    point_detail = {}
    if not args.skip_points:
        for b in (1, 64):
            k = min(steps, 64)
            pms, pkv, _ = decode_bench(runner, model, b, args.prompt_len, k, warmup, rng)
            points[f"decode_b{b}"] = b / (pms / 1e3)
            gbs = (weight_bytes + pkv) / (pms / 1e3) / 1e9
            point_detail[f"decode_b{b}"] = {"ms_per_step": pms, "achieved": gbs,
                                            "frac": gbs / pk["hbm_gbs"]}
    # the same with the page size the engine uses when it is not told one
    engine_page = None
    own = Engine.__init__.__kwdefaults__["page_size"]
    if own != args.page_size and not args.skip_points:
        del engine, runner
        torch.cuda.empty_cache()
        per_req = args.prompt_len + max(warmup, SETTLE_STEPS) + steps + ahead + own
        eng2 = Engine(model, page_size=own,
                      cache_tokens=max(args.batch * per_req, T + own),
                      token_budget=budget, max_requests=args.batch, context=context)
        p2 = prefill_record(model, prefill_bench(eng2.runner, model, T, rng), T, pk)
        d_ms, _, _ = decode_bench(eng2.runner, model, args.batch, args.prompt_len, steps, warmup,
                                  rng)
        e2, _ = e2e_bench(eng2, args.batch, args.prompt_len, steps, warmup, rng)
        engine_page = {"page_size": own, "value": args.batch / (d_ms / 1e3), "ms_per_step": d_ms,
                       "e2e": e2, "prefill_value": p2["value"], "prefill_ms": p2["ms"],
                       "prefill_frac": p2["frac"], "prefill_runs_ms": p2["runs_ms"]}
    all_clk = clocks.summary()
    name = NAMES.get(args.model, args.model)
    line = {
        "metric": "decode tok/s at batch %d (%s sizes, random bf16 weights); prefill and "
                  "batch 1 / 64 in `prefill` and `points`" % (args.batch, name), "value": value,
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, seeded random weights", "impl": "ours",
        "config": {"model": args.model, "layers": c.num_hidden_layers, "layers_full": full_layers,
                   "hidden": c.hidden_size, "heads": c.num_attention_heads,
                   "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                   "intermediate": c.intermediate_size, "vocab": c.vocab_size,
                   "global_batch": args.batch, "seq_len": args.prompt_len,
                   "context": context, "page_size": args.page_size,
                   "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights %.1f GB)" % (weight_bytes / 1e9),
                   "peaks": pk["source"], "untimed_steps": max(warmup, SETTLE_STEPS)},
        # per step the engine copies one int32 array (header, token id, position, request slot,
        # wanted row and the index of the token drawn on the device per request, block-table
        # changes) and, when the set of requests or a random draw changes them, the sampler's
        # options; it reads back four status words and one token id per request.  Counted where
        # the engine copies them.
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": copied[0],
                "d2h_bytes_per_step": copied[1]},
        "gpu_launches": launches, "clocks": clk, "clocks_whole_run": all_clk, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points, "point_detail": point_detail,
    }
    if engine_page:
        line["engine_page"] = engine_page
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
