"""Each request alone and whole: the engine's logits at every position against the plain
implementation, in 32-bit and in bfloat16."""
import pytest

from util import TINY, assert_close, model_dir, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def make_runner(name, dtype, n_tokens=512, max_requests=8):
    from llmario_b200.engine import Model, ModelRunner

    model = Model.from_folder(model_dir(name, dtype), dtype, "cuda:0")
    page = TINY[name]["page_size"]
    return ModelRunner(model, page_size=page, n_pages=-(-n_tokens // page),
                       max_requests=max_requests, max_context=n_tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts(name, dtype):
    from llmario_b200.engine import StepEntry

    runner = make_runner(name, dtype)
    for i, n in enumerate((5, 11, 17, 70)):
        toks = random_tokens(name, n, seed=100 + i)
        logits = runner.step([StepEntry(f"r{i}", toks, list(range(n)))]).cpu().numpy()
        runner.close(f"r{i}")
        assert_close(logits, plain_logits(name, dtype, toks), dtype, f"{name} {dtype} n={n}", name)
    runner.cache.check_invariants()
