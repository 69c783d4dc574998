"""Command line in the manner of the reference: ``run`` and ``bench``.

``run`` mirrors ``llmario run`` (crates/cli/src/main.rs:53-69: ``--max-tokens``,
``--temperature``, ``--context``) and ``llmario-engine raw-run``
(crates/engine/bin/src/main.rs:124-144: ``--model``, ``--tokens``, ``--n``, ``--ctx``): token
ids in, token ids out, with the prefill and decode rates on standard error as raw-run prints
them (main.rs:521-547).  ``bench`` mirrors ``llmario bench`` (crates/cli/src/bench.rs:13-60:
``--model``, ``--concurrency``, ``--runs``, ``--warmup``, ``--temperature``, ``--seed``,
``--out``).  The engine starts at token ids: there is no tokenizer, so a prompt is given as
ids or as a length of random ids.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time
from typing import Optional, Sequence

PRESETS = {
    # layer sizes of the benchmark configurations; weights are random
    "qwen3-8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                     vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                     tie_word_embeddings=False, max_position_embeddings=40960),
    "qwen3-0.6b": dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16,
                       num_key_value_heads=8, head_dim=128, intermediate_size=3072,
                       vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                       tie_word_embeddings=True, max_position_embeddings=40960),
    "qwen3-32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                      num_key_value_heads=8, head_dim=128, intermediate_size=25600,
                      vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                      tie_word_embeddings=False, max_position_embeddings=40960),
    "tiny-a": dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
                   rope_theta=1e4, rms_norm_eps=1e-6, tie_word_embeddings=True,
                   max_position_embeddings=2048),
    "tiny-b": dict(num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
                   num_key_value_heads=3, head_dim=32, intermediate_size=160, vocab_size=384,
                   rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
                   max_position_embeddings=4096),
}


def preset_config(name: str, num_layers: Optional[int] = None):
    from .config import Qwen3Config

    raw = dict(PRESETS[name.lower()], architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    if num_layers:
        raw["num_hidden_layers"] = int(num_layers)
    return Qwen3Config.from_dict(raw)


def _engine(args, max_requests: int, cache_tokens: Optional[int] = None):
    from .engine.engine import Engine

    kw = dict(dtype=args.dtype, page_size=args.page_size, token_budget=args.batch,
              max_requests=max_requests, context=args.context, cache_tokens=cache_tokens)
    if args.model.lower() in PRESETS:
        return Engine(config=preset_config(args.model, getattr(args, "layers", None)),
                      seed=args.weights_seed, **kw)
    return Engine(args.model, **kw)


def _common(p: argparse.ArgumentParser) -> None:
    p.add_argument("--context", "--ctx", type=int, default=None,
                   help="per-request context tokens (default: the model's)")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--page-size", type=int, default=64, help="tokens in a cache page")
    p.add_argument("--batch", type=int, default=512, help="token budget of one step")
    p.add_argument("--weights-seed", type=int, default=0,
                   help="seed of the random weights when the model is a preset name")
    p.add_argument("--layers", type=int, default=None,
                   help="with a preset: build only this many layers")


def cmd_run(args) -> int:
    from .sampling import SamplingParams

    if args.tokens:
        prompt = [int(t) for t in args.tokens.replace(" ", "").split(",") if t]
    else:
        rng = random.Random(args.seed or 0)
        vocab = None
    eng = _engine(args, max_requests=1,
                  cache_tokens=None if args.context is None else args.context)
    if not args.tokens:
        vocab = eng.model.vocab_size
        prompt = [rng.randrange(vocab) for _ in range(args.prompt_len)]
    n = args.max_tokens if args.max_tokens is not None else args.n
    temp = 0.0 if args.temperature is None else args.temperature
    params = SamplingParams(temperature=temp, seed=args.seed, max_tokens=n,
                            top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                            repeat_penalty=args.repeat_penalty, repeat_last_n=args.repeat_last_n,
                            presence_penalty=args.presence_penalty,
                            frequency_penalty=args.frequency_penalty)
    import torch

    rid = eng.add_request(prompt, params)
    t0 = time.perf_counter()
    first = None
    while eng.has_work():
        eng.step()
        if first is None and eng.request(rid).output:
            torch.cuda.synchronize()
            first = time.perf_counter()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    req = eng.request(rid)
    if req.error:
        print(f"error: {req.error}", file=sys.stderr)
        return 1
    out = req.output
    ttft = (first or t1) - t0
    print(f"prefill {len(prompt)} tokens in {ttft:.3f} s ({len(prompt) / max(ttft, 1e-9):.1f} "
          f"tok/s)", file=sys.stderr)
    if len(out) > 1:
        d = t1 - (first or t1)
        print(f"decode {len(out) - 1} tokens in {d:.3f} s ({(len(out) - 1) / max(d, 1e-9):.1f} "
              f"tok/s)", file=sys.stderr)
    print(f"[TTFT {ttft * 1e3:.0f} ms · {len(out)} tokens · {req.finish_reason}]",
          file=sys.stderr)
    print(",".join(str(t) for t in out))
    return 0


def cmd_bench(args) -> int:
    """Prefill and decode rates at each concurrency level, by the reference's definitions
    (docs/BENCHMARK_PLAN.md:28-42: TTFT; prefill = prompt tokens / TTFT; decode = (completion
    - 1) / (t_last - t_first); aggregate tokens per second), every run reported, as JSON and as
    a Markdown table (crates/cli/src/bench.rs:13-60 writes both), with the fraction of the memory
    roofline that the decode steps reach."""
    import torch

    from .benchmarks.roofline import decode_step_bytes, peaks
    from .sampling import SamplingParams

    levels = [int(c) for c in str(args.concurrency).split(",") if c]
    need = max(levels) * (args.prompt_len + args.decode_len + args.page_size)
    args.context = args.context or (args.prompt_len + args.decode_len + 1)
    eng = _engine(args, max_requests=max(levels), cache_tokens=need)
    vocab = eng.model.vocab_size
    pk = peaks()
    rng = random.Random(args.seed or 0)
    results = []
    for level in levels:
        runs = []
        for it in range(args.warmup + args.runs):
            prompts = [[rng.randrange(vocab) for _ in range(args.prompt_len)]
                       for _ in range(level)]
            params = SamplingParams(temperature=args.temperature, seed=args.seed,
                                    max_tokens=args.decode_len, ignore_eos=True)
            ids = [eng.add_request(p, params) for p in prompts]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            t_first = None
            decode_steps = 0
            while eng.has_work():
                eng.step()
                if t_first is None and all(eng.request(i).output for i in ids):
                    torch.cuda.synchronize()
                    t_first = time.perf_counter()
                elif t_first is not None:
                    decode_steps += 1
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            gen = sum(len(eng.request(i).output) for i in ids)
            if it >= args.warmup:
                decode_s = max(t1 - t_first, 1e-9)
                step_bytes = decode_step_bytes(eng.model, eng.runner, level,
                                               args.prompt_len + args.decode_len / 2.0)
                gbs = step_bytes * max(decode_steps, 1) / decode_s / 1e9
                runs.append({"ttft_s": t_first - t0,
                             "prefill_tok_s": level * args.prompt_len / (t_first - t0),
                             "decode_tok_s": (gen - level) / decode_s,
                             "aggregate_tok_s": gen / (t1 - t0),
                             "decode_gb_s": gbs, "decode_roofline_frac": gbs / pk["hbm_gbs"]})
        results.append({"concurrency": level, "runs": runs})
        best = max(r["decode_tok_s"] for r in runs)
        print(f"concurrency {level}: decode {best:.1f} tok/s, prefill "
              f"{max(r['prefill_tok_s'] for r in runs):.1f} tok/s", file=sys.stderr)
    report = {"model": args.model, "dtype": args.dtype, "prompt_len": args.prompt_len,
              "decode_len": args.decode_len, "page_size": args.page_size, "label": args.label,
              "peaks": pk, "results": results}
    text = json.dumps(report, indent=1)
    if args.out:
        os.makedirs(args.out, exist_ok=True)
        stem = os.path.join(args.out, args.label or "bench")
        with open(stem + ".json", "w") as f:
            f.write(text)
        with open(stem + ".md", "w") as f:
            f.write(bench_markdown(report))
    print(text)
    return 0


def bench_markdown(report: dict) -> str:
    """The report of ``bench`` as a Markdown table, one row per run."""
    pk = report["peaks"]
    lines = [f"# bench: {report['model']} ({report['dtype']})", "",
             f"Prompts of {report['prompt_len']} random token ids, {report['decode_len']} decoded "
             f"tokens each, pages of {report['page_size']}.  Memory roofline: "
             f"{pk['hbm_gbs']:.0f} GB/s ({pk['source']}).", "",
             "| concurrency | run | TTFT ms | prefill tok/s | decode tok/s | aggregate tok/s | "
             "decode GB/s | of roofline |", "|---|---|---|---|---|---|---|---|"]
    for level in report["results"]:
        for i, r in enumerate(level["runs"]):
            lines.append(f"| {level['concurrency']} | {i} | {r['ttft_s'] * 1e3:.1f} | "
                         f"{r['prefill_tok_s']:.0f} | {r['decode_tok_s']:.0f} | "
                         f"{r['aggregate_tok_s']:.0f} | {r['decode_gb_s']:.0f} | "
                         f"{r['decode_roofline_frac']:.3f} |")
    return "\n".join(lines) + "\n"


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="llmario-b200", description="Qwen3 inference engine for "
                                 "one B200: token ids in, token ids out")
    sub = ap.add_subparsers(dest="cmd", required=True)
    run = sub.add_parser("run", help="generate from a prompt of token ids")
    run.add_argument("model", help="model folder, or a preset name: " + ", ".join(PRESETS))
    run.add_argument("--tokens", default=None, help="comma-separated prompt token ids")
    run.add_argument("--prompt-len", type=int, default=16,
                     help="without --tokens: this many random ids")
    run.add_argument("--max-tokens", type=int, default=None, help="tokens to generate")
    run.add_argument("--n", type=int, default=16, help="tokens to generate (raw-run's name)")
    run.add_argument("--temperature", type=float, default=None,
                     help="0 or absent: greedy")
    run.add_argument("--seed", type=int, default=None)
    run.add_argument("--top-k", type=int, default=40)
    run.add_argument("--top-p", type=float, default=0.95)
    run.add_argument("--min-p", type=float, default=0.05)
    run.add_argument("--repeat-penalty", type=float, default=1.0,
                     help="over the last --repeat-last-n tokens, prompt included; 1 disables")
    run.add_argument("--repeat-last-n", type=int, default=64)
    run.add_argument("--presence-penalty", type=float, default=0.0)
    run.add_argument("--frequency-penalty", type=float, default=0.0)
    _common(run)
    run.set_defaults(fn=cmd_run)
    bench = sub.add_parser("bench", help="prefill and decode rates at given concurrency")
    bench.add_argument("--model", "-m", required=True)
    bench.add_argument("--concurrency", default="1,4")
    bench.add_argument("--runs", type=int, default=3)
    bench.add_argument("--warmup", type=int, default=1)
    bench.add_argument("--temperature", type=float, default=0.0)
    bench.add_argument("--seed", type=int, default=None)
    bench.add_argument("--prompt-len", type=int, default=1024)
    bench.add_argument("--decode-len", type=int, default=256)
    bench.add_argument("--label", default=None)
    bench.add_argument("--out", default=None, help="folder for the report")
    _common(bench)
    bench.set_defaults(fn=cmd_bench)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
