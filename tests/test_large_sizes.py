"""The kernels at the sizes of the benchmark model (Qwen3-8B layer sizes, two layers, random
weights): the bfloat16 path against the true 32-bit path on the same weights, whole prompts,
portions and decode steps.  The 32-bit path is checked against the plain implementation on the
tiny configurations elsewhere; here it is the reference for sizes the plain implementation is
too slow for."""
import random

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def models():
    from llmario_b200.cli import preset_config
    from llmario_b200.engine import Model
    from llmario_b200.weights import random_tensors

    cfg = preset_config("qwen3-8b", 2)
    spec = cfg.to_spec()
    w16 = random_tensors(spec, 3, torch.bfloat16, DEV)
    w32 = {k: v.float() for k, v in w16.items()}
    m16 = Model(spec, w16, torch.bfloat16, DEV)
    m32 = Model(spec, w32, torch.float32, DEV)
    w16.clear(), w32.clear()
    yield m16, m32


def test_benchmark_sizes_bfloat16_against_float32(models):
    from llmario_b200 import kernels
    from llmario_b200.engine import ModelRunner, StepEntry

    m16, m32 = models
    assert m16.blocks[0].mixer.head_dim == 128 and m16.hidden_size == 4096
    rng = random.Random(1)
    vocab = m16.vocab_size
    prompts = {"a": [rng.randrange(vocab) for _ in range(700)],     # the persistent product
               "b": [rng.randrange(vocab) for _ in range(45)],
               "c": [rng.randrange(vocab) for _ in range(130)]}
    tails = {r: [rng.randrange(vocab) for _ in range(6)] for r in prompts}

    def run(model, cut):
        runner = ModelRunner(model, page_size=16, cache_tokens=2048, max_requests=4,
                             max_context=1024, token_budget=1024)
        out = {r: [] for r in prompts}
        if cut == "whole":
            for r, toks in prompts.items():
                out[r].append(runner.step([StepEntry(r, toks, [len(toks) - 1])]).cpu().numpy())
        else:   # "a" in portions of 300 beside the others
            at = 0
            first = True
            while at < 700:
                n = min(300, 700 - at)
                entries = [StepEntry("a", prompts["a"][at:at + n], [n - 1] if at + n == 700 else [])]
                if first:
                    entries += [StepEntry(r, prompts[r], [len(prompts[r]) - 1]) for r in ("b", "c")]
                res = runner.step(entries).cpu().numpy()
                if first:
                    out["b"].append(res[-2:-1]), out["c"].append(res[-1:])
                    res = res[:-2]
                if len(res):
                    out["a"].append(res)
                at += n
                first = False
        for i in range(6):      # decode steps of all three (recorded as a graph from the second)
            res = runner.step([StepEntry(r, [tails[r][i]], [0]) for r in prompts]).cpu().numpy()
            for j, r in enumerate(prompts):
                out[r].append(res[j:j + 1])
        kernels.check_tc_status(DEV)
        assert runner.counters["graph_replays"] >= 4
        return {r: np.concatenate(v) for r, v in out.items()}

    ref = run(m32, "whole")
    ref_cut = run(m32, "portions")
    got = run(m16, "whole")
    got_cut = run(m16, "portions")
    for r in prompts:
        scale = np.abs(ref[r]).max()
        # the 32-bit path does not depend on the cut beyond the order of sums
        assert np.abs(ref_cut[r] - ref[r]).max() <= 1e-4 * max(1.0, scale), r
        for g in (got[r], got_cut[r]):
            assert np.isfinite(g).all()
            assert np.abs(g - ref[r]).max() <= 5e-2 * scale, (r, np.abs(g - ref[r]).max(), scale)
