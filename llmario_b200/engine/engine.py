"""The Python entry point: an engine that takes token ids and returns token ids.

``Engine.generate`` is the analogue of the reference's ``raw-run`` (prompt ids in, generated ids
out: crates/engine/bin/src/main.rs:459-558) on top of the continuous-batching loop of its
server (crates/engine/server/src/engine.rs:621-710).  Option names follow the reference's
``serve`` flags: ``context`` (--ctx), ``max_requests`` (--parallel), ``token_budget`` (--batch)
(crates/engine/bin/src/main.rs:31-90).
"""
from __future__ import annotations

import itertools
import time
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from .. import kernels
from ..sampling import DeviceSampler, RequestSampler, SamplingParams
from .model import Model
from .scheduler import FINISHED, Request, Scheduler, StepPlan
from .step import ModelRunner, StepEntry


class _Launched:
    """A step that is queued on the device: its plan and the tokens it will have drawn."""

    def __init__(self, plan: StepPlan, pending):
        self.plan, self.pending = plan, pending


class Engine:
    def __init__(self, model: Union[str, Model, None] = None, *, config=None, seed: int = 0,
                 dtype="bfloat16", device: str = "cuda:0", page_size: int = 64,
                 num_pages: Optional[int] = None, cache_tokens: Optional[int] = None,
                 token_budget: int = 512, max_requests: int = 64,
                 context: Optional[int] = None, num_layers: Optional[int] = None,
                 lookahead: bool = True, native: bool = True):
        """``model``: a folder with config.json and model.safetensors, or a built
        :class:`Model`; or give ``config`` (a typed configuration) and ``seed`` for random
        weights.  ``context``: most tokens of one request; ``max_requests``: requests running at
        once; ``token_budget``: most tokens in one step; ``num_pages`` / ``cache_tokens``: size
        of the cache (default: room for every request slot at full context, or what nine tenths
        of the free device memory hold, whichever is less).  ``lookahead``:
        while a step runs, the next one is already planned and queued on the device (rows whose
        input is the token in flight take it from the sampler's output there), so that the
        device does not wait for the host between steps; the tokens a caller sees are the same.
        ``native``: standard blocks are driven by the C++ step driver (one call per run of
        layers) instead of launch by launch from Python; the launches are the same."""
        if not torch.cuda.is_available():
            raise RuntimeError("llmario_b200 needs a CUDA device; there is no CPU path")
        if isinstance(model, Model):
            self.model = model
        elif model is not None:
            self.model = Model.from_folder(model, dtype, device)
        elif config is not None:
            self.model = Model.random(config, seed, dtype, device)
        else:
            raise ValueError("give a model folder, a Model, or a config for random weights")
        spec = self.model.spec
        ctx = int(context or spec.max_positions)
        self.runner = ModelRunner(self.model, page_size=page_size, n_pages=num_pages,
                                  max_requests=max_requests, max_context=ctx,
                                  token_budget=token_budget, cache_tokens=cache_tokens,
                                  use_native=native)
        self.scheduler = Scheduler(self.runner.cache, token_budget, ctx, spec.eos_token_ids)
        self.sampler = DeviceSampler(self.model.device)
        self._ids = itertools.count()
        self._requests: Dict[Any, Request] = {}
        self.timers = {"step_s": 0.0, "sample_s": 0.0}
        self.counters = {"failed_steps": 0}
        self.lookahead = bool(lookahead)
        self._flying: Optional[_Launched] = None     # a step queued ahead, not yet read

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Any = None) -> Any:
        params = params or SamplingParams()
        rid = request_id if request_id is not None else f"req-{next(self._ids)}"
        if rid in self._requests and self._requests[rid].state != FINISHED:
            raise ValueError(f"request id {rid!r} is in use")
        vocab = self.model.vocab_size
        prompt = [int(t) for t in prompt]
        for t in prompt:
            if not 0 <= t < vocab:
                raise ValueError(f"token {t} outside the vocabulary of {vocab}")
        req = Request(rid, prompt, params)
        req.sampler = RequestSampler(params, vocab)
        for t in prompt:                       # the prompt is penalised too (sampler.rs:374-386)
            req.sampler.accept(t)
        self.scheduler.add(req)
        self._requests[rid] = req
        return rid

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> List[Request]:
        """One iteration: plan, run the batch, sample, finish.  Returns requests that finished
        (or failed) in this iteration."""
        finished: List[Request] = []
        cur, self._flying = self._flying, None
        if cur is None:
            plan = self.scheduler.plan()
            finished += plan.failed
            if not plan.entries:
                return finished
            try:
                cur = self._launch(plan, None)
            except RuntimeError as e:
                # a launch of the step raised (a kernel refused a size, memory ran out): the
                # step function has put its own state right; the step's requests fail
                return finished + self._fail_plans([plan], f"step could not be launched: {e}")
        if self.lookahead:
            # queue the step after this one before waiting for this one's tokens
            ahead = self.scheduler.plan_ahead(cur.plan)
            if ahead is not None:
                try:
                    self._flying = self._launch(ahead, cur)
                except RuntimeError:
                    self._flying = None      # planned ahead only: the next iteration plans anew
        t0 = time.perf_counter()
        tokens = cur.pending.result() if cur.pending is not None else []
        self.timers["wait_s"] = self.timers.get("wait_s", 0.0) + time.perf_counter() - t0
        fault = kernels.status_message(cur.pending.status) if cur.pending is not None else None
        if fault is not None:
            return finished + self._fail_step(cur, fault)
        sampled = {}
        i = 0
        for e in cur.plan.entries:
            if e.samples:
                sampled[e.request.id] = tokens[i]
                e.request.sampler.accept(tokens[i])
                i += 1
        finished += self.scheduler.complete(cur.plan, sampled)
        return finished

    def _launch(self, plan: StepPlan, after: Optional["_Launched"]) -> "_Launched":
        """Queue the step of ``plan`` and its draw on the device.  ``after``: the step that is
        still running and whose drawn tokens are this step's input."""
        entries = []
        source = None
        row_of = {}        # request id -> its row among the tokens that ``after`` draws
        if after is not None:
            for e in after.plan.entries:
                if e.samples:
                    row_of[e.request.id] = len(row_of)
        rows: List[int] = []        # per token row: where on the device its token comes from, or -1
        inflight: List[int] = []    # per sampling row: the same for the token that enters its window
        for e in plan.entries:
            r = e.request
            want = [e.count - 1] if e.samples else []
            # the position of the token ``after`` is drawing for this request
            unknown = len(r.prompt) + len(r.output) if r.id in row_of else None
            if unknown is not None and e.start + e.count - 1 >= unknown:
                if e.count != 1 or e.start != unknown:
                    raise RuntimeError(f"request {r.id!r}: a portion planned ahead reaches past "
                                       "the token in flight")
                entries.append(StepEntry(r.id, [0], want))
                rows.append(row_of[r.id])
                if e.samples:
                    inflight.append(row_of[r.id])
            else:
                entries.append(StepEntry(r.id, r.tokens(e.start, e.count), want))
                rows += [-1] * e.count
                if e.samples:
                    inflight.append(-1)
        if any(x >= 0 for x in rows):
            source = (self.sampler.device_tokens, rows)
        t0 = time.perf_counter()
        logits = self.runner.step(entries, source)
        samplers = [e.request.sampler for e in plan.entries if e.samples]
        t1 = time.perf_counter()
        pending = self.sampler.launch(logits, samplers, inflight) if samplers else None
        t2 = time.perf_counter()
        self.timers["step_s"] += t1 - t0
        self.timers["sample_s"] += t2 - t1
        return _Launched(plan, pending)

    def _fail_step(self, cur: "_Launched", fault: str) -> List[Request]:
        """A kernel of the step reported a failure through the status words (a bounded wait
        that gave up, a token id outside the table): what the step computed cannot be trusted.
        Its requests end with ``finish_reason == "error"`` instead of receiving tokens drawn
        from such logits (the reference's ``Event::Error``, engine.rs:1140); so do the requests
        of a step already queued behind it, which ran on the same state.  The status words are
        cleared and recorded steps are dropped, so the engine can take new requests."""
        plans = [cur.plan] + ([self._flying.plan] if self._flying is not None else [])
        if self._flying is not None and self._flying.pending is not None:
            self._flying.pending.result()          # let the step ahead leave the device
        self._flying = None
        torch.cuda.current_stream().synchronize()
        kernels.clear_status(self.model.device)
        self.runner.drop_buffers()         # a buffer kept at zero may hold partial sums
        return self._fail_plans(plans, f"step failed on the device: {fault}")

    def _fail_plans(self, plans: Sequence[StepPlan], message: str) -> List[Request]:
        """End every request of ``plans`` that is still running with ``finish_reason ==
        "error"``; their pages are given back."""
        failed: List[Request] = []
        for plan in plans:
            for e in plan.entries:
                if e.request.state != FINISHED:
                    self.scheduler.fail(e.request, message)
                    failed.append(e.request)
        self.counters["failed_steps"] += 1
        return failed

    def abort(self, request_id: Any) -> None:
        """Drop a request wherever it is; a step already queued for it runs to its end and its
        result is ignored."""
        self.scheduler.abort(self._requests[request_id])

    def run_until_done(self) -> List[Request]:
        done: List[Request] = []
        while self.has_work():
            done += self.step()
        return done

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[List[int]]:
        """Generated token ids for every prompt (host lists in, host lists out)."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        self.run_until_done()
        out = []
        for rid in ids:
            r = self.release(rid)
            if r.error:
                raise RuntimeError(f"request {rid!r}: {r.error}")
            out.append(list(r.output))
        return out

    def request(self, request_id: Any) -> Request:
        return self._requests[request_id]

    def release(self, request_id: Any) -> Optional[Request]:
        """Forget a finished request (its record is kept until then so that its output can be
        read).  Returns the record, or None when the id is unknown."""
        r = self._requests.get(request_id)
        if r is not None and r.state != FINISHED:
            raise ValueError(f"request {request_id!r} is still {r.state}")
        return self._requests.pop(request_id, None)

    def stats(self) -> Dict[str, Any]:
        """Counters in the spirit of the reference's ``Stats`` (engine.rs:59-159)."""
        c = self.runner.cache
        return {**self.runner.counters, **self.scheduler.counters, **self.counters,
                "h2d_bytes": self.runner.counters["h2d_bytes"] + self.sampler.h2d_bytes,
                "d2h_bytes": self.sampler.d2h_bytes,
                "cache": dict(c.counters), "free_pages": c.free_pages(),
                "pages": [g.n_pages for g in c.groups], "running": len(self.scheduler.running),
                "waiting": len(self.scheduler.waiting), **self.timers}
