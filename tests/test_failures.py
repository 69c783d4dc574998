"""A failure on the device is a failed request, not a wrong token.

The TMA / tcgen05 kernels bound every wait; a wait that gives up records its role in the
library's status words, and the embedding kernel records a token id outside its table there.
The words travel to the host with every step's drawn tokens.  These tests make both happen
without a kernel that misbehaves: a self-test kernel whose only job is to wait a few
microseconds on a barrier at which nothing arrives, give up and return; and a token id patched
in on the device."""
import pytest
import torch

from util import TINY, model_dir, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_a_wait_that_gives_up_is_recorded_and_raised():
    from llmario_b200 import kernels

    kernels.check_tc_status(DEV)                       # clean to begin with
    kernels.selftest_wait_gives_up(DEV, limit_cycles=20000)
    torch.cuda.synchronize()
    assert kernels.status_words(DEV)[0].item() == 99   # the role the kernel recorded
    with pytest.raises(kernels.KernelError, match="gave up waiting.*role 99"):
        kernels.check_tc_status(DEV)
    kernels.check_tc_status(DEV)                       # raised once, cleared


@pytest.mark.parametrize("lookahead", [False, True])
def test_the_engine_fails_the_requests_of_a_step_whose_kernel_gave_up(lookahead):
    from llmario_b200 import Engine, SamplingParams, kernels

    name, dtype = "D", "bfloat16"
    params = SamplingParams(temperature=0.0, max_tokens=12)
    prompts = [random_tokens(name, n, 60 + n) for n in (9, 21, 5)]

    def engine():
        return Engine(model_dir(name, dtype), dtype=dtype, page_size=16, cache_tokens=512,
                      max_requests=4, context=128, token_budget=64, lookahead=lookahead)

    want = engine().generate(prompts, params)
    eng = engine()
    ids = [eng.add_request(p, params) for p in prompts[:2]]
    for _ in range(4):
        assert eng.step() == []
    kernels.selftest_wait_gives_up(DEV)                # "a kernel of the next step gave up"
    finished = []
    for _ in range(3):
        finished += eng.step()
        if finished:
            break
    assert sorted(r.id for r in finished) == sorted(ids)
    for r in finished:
        assert r.finish_reason == "error" and "gave up waiting" in r.error
        assert 0 < len(r.output) < 12                  # what it had before the failure is kept
    st = eng.stats()
    assert st["failed_steps"] == 1 and st["failed"] == 2 and not eng.has_work()
    assert st["free_pages"] == st["pages"]
    eng.runner.cache.check_invariants()
    kernels.check_tc_status(DEV)                       # the engine cleared the words
    # and the engine goes on: new requests get the tokens a fresh engine gives them
    assert eng.generate(prompts, params) == want
    with pytest.raises(RuntimeError, match="step failed on the device"):
        ids = [eng.add_request(p, params) for p in prompts[:1]]
        eng.step()
        kernels.selftest_wait_gives_up(DEV)
        eng.generate(prompts[1:2], params)


def test_a_token_id_outside_the_table_is_reported_with_its_row():
    """The step function refuses bad ids on the host; an id that only exists on the device (a
    token patched in from the sampler's buffer) is caught by the embedding kernel."""
    from llmario_b200 import kernels
    from llmario_b200.engine import Model, ModelRunner, StepEntry

    name = "B"
    model = Model.from_folder(model_dir(name, "float32"), "float32", DEV)
    runner = ModelRunner(model, page_size=8, n_pages=8, max_requests=2, max_context=32)
    source = torch.tensor([3, TINY[name]["vocab_size"] + 5], dtype=torch.int32, device=DEV)
    runner.step([StepEntry("a", [1, 2, 3], []), StepEntry("b", [4, 5], [])],
                device_tokens=(source, [-1, 0, -1, -1, 1]))
    with pytest.raises(kernels.KernelError, match="outside the embedding table at row 4"):
        kernels.check_tc_status(DEV)
    kernels.check_tc_status(DEV)


def test_a_launch_that_raises_leaves_the_runner_usable(monkeypatch):
    """A launch inside the step raises (here: the head's product, made to fail once).  The
    requests have not advanced, block-table changes of the failed step are applied by the next
    one, and the logits of the repeated step are those of an undisturbed runner."""
    from llmario_b200 import kernels
    from llmario_b200.engine import Model, ModelRunner, StepEntry
    from util import plain_logits, assert_close

    name, dtype = "D", "bfloat16"
    model = Model.from_folder(model_dir(name, dtype), dtype, DEV)
    runner = ModelRunner(model, page_size=16, n_pages=16, max_requests=2, max_context=128)
    toks = random_tokens(name, 40, 77)
    runner.step([StepEntry("a", toks[:14], [])])
    real = model.head.forward
    state = {"fail": True}

    def flaky(ctx, h, logits):
        if state["fail"]:
            state["fail"] = False
            raise kernels.KernelError("made to fail")
        return real(ctx, h, logits)

    monkeypatch.setattr(model.head, "forward", flaky)
    entries = [StepEntry("a", toks[14:33], list(range(19))), StepEntry("b", toks[:5], [4])]
    with pytest.raises(kernels.KernelError, match="made to fail"):
        runner.step(entries)                 # crosses a page edge: new table cells were taken
    assert runner.length("a") == 14 and not runner.cache.has("b")
    assert runner.counters["failed_launches"] == 1
    got = runner.step(entries).cpu().numpy()
    ref = plain_logits(name, dtype, toks)
    assert_close(got[:19], ref[14:33], dtype, "after a failed launch", name)
    assert_close(got[19:], ref[4:5], dtype, "after a failed launch, new request", name)
    runner.cache.check_invariants()


@pytest.mark.parametrize("lookahead", [False, True])
def test_the_engine_fails_the_requests_of_a_step_that_could_not_be_launched(monkeypatch, lookahead):
    """A launch raises inside the step function (made to, once).  When it is the step the engine
    needs next, the engine ends that step's requests with an error and goes on; later requests
    get the tokens a fresh engine gives them.  When it is a step that was only being queued
    ahead, nothing is lost: the engine plans that step again in its turn."""
    from llmario_b200 import Engine, SamplingParams, kernels

    name, dtype = "D", "bfloat16"
    params = SamplingParams(temperature=0.0, max_tokens=10)
    prompts = [random_tokens(name, n, 80 + n) for n in (12, 30)]

    def engine():
        return Engine(model_dir(name, dtype), dtype=dtype, page_size=16, cache_tokens=512,
                      max_requests=4, context=128, token_budget=64, lookahead=lookahead)

    want = engine().generate(prompts, params)
    eng = engine()
    ids = [eng.add_request(p, params) for p in prompts]
    for _ in range(3):
        assert eng.step() == []
    real = eng.runner._graph_step          # (decode steps are replayed: no part's forward runs)
    state = {"fail": True}

    def flaky(key, forward):
        if state["fail"]:
            state["fail"] = False
            raise kernels.KernelError("made to fail")
        return real(key, forward)

    monkeypatch.setattr(eng.runner, "_graph_step", flaky)
    finished = eng.run_until_done()
    assert sorted(r.id for r in finished) == sorted(ids) and not state["fail"]
    st = eng.stats()
    if lookahead:
        assert [eng.request(i).output for i in ids] == want
        assert all(r.finish_reason == "length" for r in finished)
    else:
        assert all(r.finish_reason == "error" and "made to fail" in r.error for r in finished)
        assert all(0 < len(r.output) < 10 for r in finished)
    assert st["failed_launches"] == 1 and st["failed_steps"] == (0 if lookahead else 1)
    assert st["free_pages"] == st["pages"] and not eng.has_work()
    eng.runner.cache.check_invariants()
    for i in ids:
        eng.release(i)
    assert eng.generate(prompts, params) == want
