#!/usr/bin/env python3
"""Decode and prefill rates of the engine on one B200, as one JSON line.

    python bench.py --gpus 1 --steps K --warmup W

A "step" is one decode step of a batch of requests.  The default run has the layer sizes of
Qwen3-8B with seeded random bfloat16 weights, 8 requests with 1,024-token prompts of uniform
random ids, context 8,192, pages of 16 tokens (the named configuration).  ``value`` is decoded
tokens per second timed on the device around K consecutive steps of the step function plus the
sampling kernel; ``e2e`` is the same through ``Engine.step`` with host token lists in and out.
``engine_page`` repeats prefill, ``value`` and ``e2e`` with the engine's default page of 64 tokens.  The weights (about 15 GB)
are larger than the L2 cache, so no flush is needed between steps.
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

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

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

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
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


def reference_arm():
    """The reference is a Rust workspace (no Python package, no setup.py / pyproject.toml) and
    there is no Rust toolchain in the image, so it cannot be installed or run here."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "mannysinghx/LLMario is a Rust workspace without a Python package: pip "
                      "cannot install it, no cargo/rustc offline, and it has no CUDA backend"}))
    return 0


def decode_bench(runner, sampler, model, batch, prompt_len, steps, warmup, rng, chunk=2048):
    """Prefill ``batch`` requests of ``prompt_len`` tokens, then time ``steps`` decode steps on
    the device.  Returns (ms per step, cache bytes read per step on average)."""
    import torch

    from llmario_b200 import kernels
    from llmario_b200.engine import StepEntry
    from llmario_b200.sampling import RequestSampler, SamplingParams

    vocab = model.vocab_size
    ids = [f"b{batch}-{i}" for i in range(batch)]
    for rid in ids:
        toks = [rng.randrange(vocab) for _ in range(prompt_len)]
        for at in range(0, prompt_len, chunk):
            runner.step([StepEntry(rid, toks[at:at + chunk], [])])
    samplers = [RequestSampler(SamplingParams(temperature=0.0), vocab) for _ in ids]
    feed = [[rng.randrange(vocab) for _ in ids] for _ in range(warmup + steps)]

    def one(i):
        logits = runner.step([StepEntry(rid, [feed[i][j]], [0]) for j, rid in enumerate(ids)])
        kernels.sample(logits, sampler_bufs["t"], sampler_bufs["k"], sampler_bufs["p"],
                       sampler_bufs["m"], sampler_bufs["u"], sampler_bufs["o"])

    dev = model.device
    sampler_bufs = {"t": torch.zeros(batch, device=dev), "k": torch.zeros(batch, dtype=torch.int32, device=dev),
                    "p": torch.ones(batch, device=dev), "m": torch.zeros(batch, device=dev),
                    "u": torch.zeros(batch, dtype=torch.float64, device=dev),
                    "o": torch.zeros(batch, dtype=torch.int32, device=dev)}
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
    kv_per_token = runner.cache.storage_bytes(model.dtype) // (
        runner.cache.groups[0].n_pages * runner.page_size)
    mean_len = prompt_len + warmup + (steps - 1) / 2.0 + 1
    kv_bytes = batch * mean_len * kv_per_token
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
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n0 = sum(len(engine.request(i).output) for i in ids)
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    n1 = sum(len(engine.request(i).output) for i in ids)
    for i in ids:
        engine.abort(i)
    return (n1 - n0) / (t1 - t0)


def prefill_bench(runner, model, tokens, rng, reps=3):
    import torch

    from llmario_b200.engine import StepEntry

    vocab = model.vocab_size
    best = None
    for r in range(reps + 1):
        toks = [rng.randrange(vocab) for _ in range(tokens)]
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(f"p{r}", toks, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.close(f"p{r}")
        ms = start.elapsed_time(end)
        if r > 0:
            best = ms if best is None else min(best, ms)
    return best


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--layers", type=int, default=None, help="build fewer layers (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--page-size", type=int, default=16,
                    help="tokens in a cache page for the headline numbers (the named configuration "
                         "has 16; the engine's own default, 64, is measured too and reported "
                         "under `engine_page`)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    import torch

    from llmario_b200 import kernels
    from llmario_b200.cli import PRESETS, preset_config
    from llmario_b200.engine import Model, ModelRunner
    from llmario_b200.engine.engine import Engine
    from llmario_b200.sampling import DeviceSampler

    warmup = max(3, args.warmup)
    steps = args.steps
    pk = peaks()
    cfg = preset_config(args.model, args.layers)
    full_layers = PRESETS[args.model]["num_hidden_layers"]
    rng = random.Random(0)
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    max_batch = args.batch if args.skip_points else max(args.batch, 64)
    budget = max(2048, args.prefill_tokens)
    # room for the prompt, the decoded tokens and the tokens a request decodes while the prompts
    # of the others are still being prefilled
    ahead = args.batch * -(-args.prompt_len // budget) + 2
    per_req = args.prompt_len + warmup + steps + ahead + args.page_size
    cache_tokens = max(max_batch * per_req, args.prefill_tokens + args.page_size)
    engine = Engine(model, page_size=args.page_size, cache_tokens=cache_tokens,
                    token_budget=budget, max_requests=max_batch,
                    context=args.context)
    runner = engine.runner
    sampler = DeviceSampler(model.device)
    weight_bytes = model.weight_bytes()

    # prefill first: it also warms every kernel
    prefill_ms = prefill_bench(runner, model, args.prefill_tokens, rng)
    c = cfg
    lin = weight_bytes / 2 - c.vocab_size * c.hidden_size   # parameters of the layer matrices
    T = args.prefill_tokens
    flops = 2.0 * T * lin + 2.0 * T * T * c.num_attention_heads * c.head_dim * \
        c.num_hidden_layers + 2.0 * c.vocab_size * c.hidden_size
    prefill = {"value": T / (prefill_ms / 1e3), "tokens": T, "ms": prefill_ms,
               "frac": flops / (prefill_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)}

    clocks = ClockSampler()
    clocks.start()
    ms, kv_bytes, launches = decode_bench(runner, sampler, model, args.batch, args.prompt_len,
                                          steps, warmup, rng)
    clk = clocks.stop()
    value = args.batch / (ms / 1e3)
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9
    e2e = e2e_bench(engine, args.batch, args.prompt_len, steps, warmup, rng)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            k = min(steps, 64)
            pms, _, _ = decode_bench(runner, sampler, model, b, args.prompt_len, k, warmup, rng)
            points[f"decode_b{b}"] = b / (pms / 1e3)
    # the same with the page size the engine uses when it is not told one
    engine_page = None
    own = Engine.__init__.__kwdefaults__["page_size"]
    if own != args.page_size and not args.skip_points:
        del engine, runner
        torch.cuda.empty_cache()
        per_req = args.prompt_len + warmup + steps + ahead + own
        eng2 = Engine(model, page_size=own,
                      cache_tokens=max(args.batch * per_req, args.prefill_tokens + own),
                      token_budget=budget, max_requests=args.batch,
                      context=args.context)
        p_ms = prefill_bench(eng2.runner, model, args.prefill_tokens, rng)
        d_ms, _, _ = decode_bench(eng2.runner, sampler, model, args.batch, args.prompt_len, steps,
                                  warmup, rng)
        e2 = e2e_bench(eng2, args.batch, args.prompt_len, steps, warmup, rng)
        engine_page = {"page_size": own, "value": args.batch / (d_ms / 1e3), "ms_per_step": d_ms,
                       "e2e": e2, "prefill_value": T / (p_ms / 1e3), "prefill_ms": p_ms}

    line = {
        "metric": "decode tok/s at batch %d (Qwen3-8B sizes, random bf16 weights); prefill and "
                  "batch 1 / 64 in `prefill` and `points`" % args.batch, "value": value,
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, seeded random weights", "impl": "ours",
        "config": {"model": args.model, "layers": c.num_hidden_layers, "layers_full": full_layers,
                   "hidden": c.hidden_size, "heads": c.num_attention_heads,
                   "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                   "intermediate": c.intermediate_size, "vocab": c.vocab_size,
                   "global_batch": args.batch, "seq_len": args.prompt_len,
                   "context": args.context, "page_size": args.page_size,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 15 GB)",
                   "peaks": pk["source"]},
        # per step the engine copies one int32 array (header, token id, position, request slot,
        # wanted row and the index of the token drawn on the device per request, block-table
        # changes) and the sampler's options
        # (10 float32 words per row capacity of 64), and reads back one token id per request
        "e2e": {"value": e2e, "unit": "tokens/s",
                "h2d_bytes_per_step": 4 * (16 + 5 * ((args.batch + 3) // 4 * 4)) + 4 * 10 * 64,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches, "clocks": clk, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
    if engine_page:
        line["engine_page"] = engine_page
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
