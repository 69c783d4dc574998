"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the same
:class:`Model` and :class:`ModelRunner` that generation uses and calls ``step``.

Input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted the logits at the wanted places are written to
``<out>/<step>.f32`` as little-endian float32 ``[wanted, vocab]``; after every step a line
``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional, Sequence

import numpy as np


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each request's "
                         "count rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=64, help="tokens in a cache page")
    ap.add_argument("--max-requests", type=int, default=8, help="request slots")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.page_size <= 0 or 64 % args.page_size != 0 and args.page_size % 64 != 0:
        ap.error("--page-size must divide 64 or be a multiple of it")

    import torch

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is available; this engine has no CPU path",
              file=sys.stderr)
        return 3
    from .model import Model
    from .step import ModelRunner, StepEntry

    os.makedirs(args.out, exist_ok=True)
    model = Model.from_folder(args.model, args.dtype, args.device)
    page = args.page_size
    n_pages = -(-args.max_tokens // page)
    runner = ModelRunner(model, page_size=page, n_pages=n_pages,
                         max_requests=args.max_requests,
                         max_context=min(model.spec.max_positions, n_pages * page),
                         token_budget=args.max_tokens)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec["entries"]]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                arr = logits.cpu().numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", ()):
            runner.close(rid)
        torch.cuda.synchronize()
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
