"""The command line itself, run as a program: ``run`` (token ids in, token ids out, rates on
standard error, as the reference's raw-run: crates/engine/bin/src/main.rs:459-558) and ``bench``
(JSON and Markdown with the roofline fraction, as crates/cli/src/bench.rs:13-60 writes both)."""
import json
import os
import subprocess
import sys
import tempfile

import pytest

from util import TINY, check_greedy_against_plain, model_dir, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "bin", "llmario-b200")


def cli(*args, timeout=600):
    p = subprocess.run([sys.executable, CLI, *[str(a) for a in args]], capture_output=True,
                       text=True, timeout=timeout)
    assert p.returncode == 0, p.stderr[-3000:]
    return p


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "bfloat16")])
def test_run_prints_the_greedy_continuation(name, dtype):
    prompt = random_tokens(name, 23, 31)
    p = cli("run", model_dir(name, dtype), "--tokens", ",".join(map(str, prompt)),
            "--max-tokens", 8, "--dtype", dtype, "--page-size", TINY[name]["page_size"],
            "--context", 128)
    out = [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]
    assert len(out) == 8
    assert check_greedy_against_plain(name, dtype, prompt, out, f"run {name} {dtype}") >= 2
    # both rates and the closing line on standard error, nothing but ids on standard output
    assert "prefill 23 tokens" in p.stderr and "decode 7 tokens" in p.stderr
    assert "[TTFT" in p.stderr and "8 tokens" in p.stderr and "length" in p.stderr


def test_run_with_a_seed_is_reproducible():
    args = ("run", "tiny-a", "--prompt-len", 5, "--seed", 1, "--temperature", 0.7, "--n", 12,
            "--dtype", "float32", "--page-size", 4, "--context", 64)
    a, b = cli(*args), cli(*args)
    ids = a.stdout.strip().splitlines()[-1]
    assert ids == b.stdout.strip().splitlines()[-1] and len(ids.split(",")) == 12
    other = cli(*args[:5], 2, *args[6:])
    assert other.stdout.strip().splitlines()[-1] != ids          # another seed, other tokens
    # the penalties of the chain are options too (steps queued ahead count the token in flight)
    greedy = ("run", "tiny-a", "--prompt-len", 5, "--n", 24, "--dtype", "float32", "--page-size", 4,
              "--context", 64)
    plain_ids = cli(*greedy).stdout.strip().splitlines()[-1].split(",")
    pen = cli(*greedy, "--repeat-penalty", 1.5, "--frequency-penalty", 1.0, "--repeat-last-n", 8)
    pen_ids = pen.stdout.strip().splitlines()[-1].split(",")
    assert len(pen_ids) == 24 and pen_ids != plain_ids
    assert max(pen_ids.count(t) for t in pen_ids) <= max(plain_ids.count(t) for t in plain_ids)


def test_bench_writes_json_and_markdown_with_the_roofline_fraction():
    with tempfile.TemporaryDirectory() as d:
        p = cli("bench", "--model", "tiny-b", "--concurrency", "1,4", "--runs", 2, "--warmup", 1,
                "--prompt-len", 40, "--decode-len", 12, "--page-size", 8, "--dtype", "float32",
                "--out", d, "--label", "tiny")
        with open(os.path.join(d, "tiny.json")) as f:
            rep = json.load(f)
        assert json.loads(p.stdout) == rep
        assert [r["concurrency"] for r in rep["results"]] == [1, 4]
        for level in rep["results"]:
            assert len(level["runs"]) == 2
            for r in level["runs"]:
                assert r["ttft_s"] > 0 and r["prefill_tok_s"] > 0 and r["decode_tok_s"] > 0
                assert 0 < r["decode_roofline_frac"] < 1.2 and r["aggregate_tok_s"] > 0
        assert rep["peaks"]["source"] in ("measured", "fallback")
        with open(os.path.join(d, "tiny.md")) as f:
            md = f.read()
        assert "of roofline" in md and md.count("\n| ") >= 4 and "tiny-b" in md
