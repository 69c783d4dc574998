"""Builders of replay traces (lists of steps in the format of bin/trace_run) and a checker that
compares what a replay returned with the plain implementation."""
from __future__ import annotations

import random
from typing import Dict, List, Sequence, Tuple

import numpy as np

from util import assert_close, plain_logits


def whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, one after the other."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks,
                                              "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def bulk_then_tail(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for j in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": [toks[j]], "want": [0]}],
                "end": [rid] if j == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (16, 7, 5, 3, 2, 9, 2, 31)
             ) -> List[dict]:
    """Each request in portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                "end": [rid] if at + n == len(toks) else []})
            at += n
    return steps


def mixed(requests: Dict[str, List[int]], live: int = 4, seed: int = 0, chunk: int = 16,
          decode_tail: int = 12) -> List[dict]:
    """Up to ``live`` requests at a time: portions of some prompts beside single tokens of
    others; a request that ends makes room (and pages) for the next one.  A request may sit
    out a step."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    active: Dict[str, Tuple[List[int], int]] = {}
    steps = []
    while waiting or active:
        while waiting and len(active) < live:
            rid, toks = waiting.pop(0)
            active[rid] = (toks, 0)
        entries, ended = [], []
        for rid in list(active):
            toks, at = active[rid]
            if len(active) > 1 and rng.random() < 0.2:
                continue        # left out of this step, goes on later
            left = len(toks) - at
            if left > decode_tail:
                n = min(left - decode_tail, rng.choice([2, 3, 5, chunk, chunk]))
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            at += n
            if at == len(toks):
                ended.append(rid)
                del active[rid]
            else:
                active[rid] = (toks, at)
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def peak_tokens(steps: List[dict], round_to: int = 64) -> int:
    """Most tokens that live requests hold at any time, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def check(steps: List[dict], results: Dict[int, np.ndarray], requests: Dict[str, List[int]],
          name: str, dtype: str, what: str) -> None:
    """Every wanted row of every step against the plain logits of its request and position."""
    ref = {rid: plain_logits(name, dtype, toks) for rid, toks in requests.items()}
    at = {rid: 0 for rid in requests}
    for s in steps:
        rows = []
        for e in s["entries"]:
            rows += [ref[e["id"]][at[e["id"]] + w] for w in e["want"]]
            at[e["id"]] += len(e["tokens"])
        if rows:
            got = results[s["step"]]
            assert_close(got, np.stack(rows), dtype, f"{what} step {s['step']}", name)
    for rid, toks in requests.items():
        assert at[rid] == len(toks), f"trace did not feed all of {rid}"
