"""A plain model of the scheduler, in Python: admits requests, cuts prompts into portions under
a token budget, decodes, finishes and frees.  The engine's scheduler makes these decisions in
native code (llmario_b200/csrc/host/sched_core.cpp); a test drives both with the same random load
and wants the same plans.  It works on any cache object with the manager's query methods.

Rules, after the reference's step loop (crates/engine/server/src/engine.rs:621-710, 780-994):

* waiting requests are served first come, first served, while a request slot is free;
* a step first gives one token to every running request that is decoding, then fills what is
  left of the token budget with prompt portions, oldest request first; the last portion of one
  prompt may share a step with the first portion of the next (engine.rs:893-911);
* a request finishes on an end-of-sequence token ("stop"), after ``max_tokens`` generated tokens
  or when its context is full ("length") (engine.rs:1185-1216).

When pages run out (the reference fails the newest job, engine.rs:940-963; its unused policy
crate retracts a running request and recomputes it later, crates/engine/sched/src/lib.rs:
148-174): first prompt portions are shortened or left out of the step; if even the decoding
requests do not fit, the most recently admitted running request is preempted: its pages are
given back and it returns to the head of the waiting queue with its prompt extended by what it
has generated, to be recomputed once all of it fits the free pages.  A request that cannot fit
even alone is failed with "KV cache full".
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Sequence


WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    id: Any
    prompt: List[int]
    params: Any
    arrival: int = 0
    state: str = WAITING
    output: List[int] = field(default_factory=list)
    computed: int = 0            # tokens of prompt + output whose keys are in the cache
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    preemptions: int = 0
    sampler: Any = None

    @property
    def sequence_len(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_at(self, i: int) -> int:
        n = len(self.prompt)
        return self.prompt[i] if i < n else self.output[i - n]

    def tokens(self, start: int, n: int) -> List[int]:
        p = len(self.prompt)
        if start >= p:
            return self.output[start - p:start - p + n]
        if start + n <= p:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.output[:start + n - p]


@dataclass
class PlanEntry:
    request: Request
    start: int        # first token of the sequence fed in this step
    count: int
    samples: bool     # the step's last token is the sequence's last: its logits are sampled


@dataclass
class StepPlan:
    entries: List[PlanEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)

    @property
    def tokens(self) -> int:
        return sum(e.count for e in self.entries)


class PlainScheduler:
    def __init__(self, cache: Any, token_budget: int = 512, max_context: Optional[int]
                 = None, eos_token_ids: Sequence[int] = ()):
        if token_budget <= 0:
            raise ValueError("token_budget must be positive")
        self.cache = cache
        self.token_budget = int(token_budget)
        self.max_context = int(max_context or cache.max_context)
        self.eos = frozenset(int(e) for e in eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []      # in order of admission
        self._arrivals = itertools.count()
        self.counters = {"admitted": 0, "finished": 0, "preemptions": 0, "failed": 0,
                         "steps_planned": 0, "prompt_tokens": 0, "decode_tokens": 0}
        self._fly: dict = {}

    # ------------------------------------------------------------------ queue
    def add(self, request: Request) -> None:
        """Queue a request.  An empty prompt, or one that leaves no room in the context, is
        refused (engine.rs:788-798)."""
        if not request.prompt:
            raise ValueError("empty prompt")
        if len(request.prompt) >= self.max_context:
            raise ValueError(f"prompt of {len(request.prompt)} tokens does not fit the context "
                             f"of {self.max_context}")
        request.arrival = next(self._arrivals)
        request.state = WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _pages_for(self, req: Request, count: int, opened: bool) -> List[int]:
        if opened and self.cache.has(req.id):
            return self.cache.pages_needed(req.id, count)
        ps = self.cache.page_size
        return [-(-count // ps)] * len(self.cache.groups)

    # A request as it will stand when the step that is still running ends without an
    # end-of-sequence token (``_fly``: request id -> (tokens, draws a token) of that step; empty
    # except while the step after it is being planned).
    def _done(self, r: Request) -> int:
        return r.computed + self._fly.get(r.id, (0, 0))[0]

    def _outs(self, r: Request) -> int:
        return len(r.output) + self._fly.get(r.id, (0, 0))[1]

    def _seq(self, r: Request) -> int:
        return len(r.prompt) + self._outs(r)

    def plan(self, ahead: bool = False) -> Optional[StepPlan]:
        """Decide the next step.  Changes the queues (admission, preemption, failure) but feeds
        nothing: the caller runs the step and reports back with :meth:`complete`.  ``ahead``:
        the plan is made while a step is still running; where a request would have to give way
        or nothing could run the answer is None and nothing has changed."""
        plan = StepPlan()
        cache = self.cache
        while True:
            free = list(cache.free_pages())
            used = 0
            entries: List[PlanEntry] = []
            ok = True
            # 1. decoding requests, one token each
            for r in self.running:
                if self._done(r) == self._seq(r) - 1 and self._outs(r) > 0:
                    if ahead:
                        if self._outs(r) >= r.params.max_tokens or \
                                self._seq(r) >= self.max_context:
                            continue          # its last token is the one in flight
                    need = self._pages_for(r, 1, True)
                    if used >= self.token_budget:
                        break
                    if any(n > f for n, f in zip(need, free)):
                        if ahead:
                            return None       # someone has to go: decided with all facts known
                        ok = False
                        break
                    free = [f - n for f, n in zip(free, need)]
                    entries.append(PlanEntry(r, self._done(r), 1, True))
                    used += 1
            if not ok:
                victim = self.running[-1]
                if len(self.running) == 1:
                    self._fail(victim, "KV cache full: the request does not fit the cache "
                                       "even alone")
                    plan.failed.append(victim)
                else:
                    self._preempt(victim)
                    plan.preempted.append(victim)
                continue
            # 2. prompt portions of running requests, oldest first
            for r in self.running:
                if used >= self.token_budget:
                    break
                if self._outs(r) > 0 and self._done(r) == self._seq(r) - 1:
                    continue
                left = self._seq(r) - self._done(r)
                n = min(left, self.token_budget - used)
                n = self._fit(r, n, free, True)
                if n <= 0:
                    continue
                need = self._pages_for(r, n, True)
                free = [f - k for f, k in zip(free, need)]
                entries.append(PlanEntry(r, self._done(r), n, self._done(r) + n == self._seq(r)))
                used += n
            # 3. admission
            while self.waiting and used < self.token_budget and \
                    cache.free_slots() - self._planned_new(entries) > 0:
                r = self.waiting[0]
                left = r.sequence_len - r.computed
                if r.preemptions:
                    # a request that lost its pages comes back only when all of it fits:
                    # otherwise it would take the pages the older requests are about to need
                    # and be preempted again
                    if plan.preempted or any(
                            k > f for k, f in zip(self._pages_for(r, left + 1, False), free)):
                        break
                n = self._fit(r, min(left, self.token_budget - used), free, False)
                if n <= 0:
                    break
                self.waiting.popleft()
                r.state = RUNNING
                self.running.append(r)
                self.counters["admitted"] += 1
                need = self._pages_for(r, n, False)
                free = [f - k for f, k in zip(free, need)]
                entries.append(PlanEntry(r, r.computed, n, r.computed + n == r.sequence_len))
                used += n
            if not entries and ahead:
                return None
            if not entries and self.running:
                # nothing fits although requests are running: a prompt portion is stuck for
                # want of pages.  Make room by preempting the newest, or fail a lone request.
                victim = self.running[-1]
                if len(self.running) == 1:
                    self._fail(victim, "KV cache full: the request does not fit the cache "
                                       "even alone")
                    plan.failed.append(victim)
                else:
                    self._preempt(victim)
                    plan.preempted.append(victim)
                continue
            if not entries and self.waiting and not self.running:
                r = self.waiting.popleft()
                self._fail(r, "KV cache full: the request does not fit the cache even alone")
                plan.failed.append(r)
                continue
            plan.entries = entries
            break
        self.counters["steps_planned"] += 1
        return plan

    def plan_ahead(self, flying: StepPlan) -> Optional[StepPlan]:
        """The step after ``flying``, decided while ``flying`` is still running and the tokens it
        draws are unknown, or None when that step cannot be known yet: the planner runs on the
        requests as they will stand when ``flying`` ends without an end-of-sequence token.  A
        request that does end on such a token has a row too many in the step ahead;
        :meth:`complete` passes over it.  The cache lengths already count ``flying``."""
        if flying.preempted or flying.failed or not flying.entries:
            return None
        self._fly = {e.request.id: (e.count, int(e.samples)) for e in flying.entries
                     if e.request.state == RUNNING}
        try:
            plan = self.plan(ahead=True)
        finally:
            self._fly = {}
        if plan is not None:
            self.counters["steps_planned_ahead"] = self.counters.get("steps_planned_ahead", 0) + 1
        return plan

    def _planned_new(self, entries: List[PlanEntry]) -> int:
        return sum(1 for e in entries if not self.cache.has(e.request.id))

    def _fit(self, r: Request, n: int, free: List[int], opened: bool) -> int:
        """Largest count <= n whose pages fit in ``free``."""
        if n <= 0:
            return 0
        opened = opened and self.cache.has(r.id)
        need = self._pages_for(r, n, opened)
        if all(k <= f for k, f in zip(need, free)):
            return n
        ps = self.cache.page_size
        have = self.cache.length(r.id) if opened else 0
        held = len(self.cache.pages_of(r.id, 0)) if opened and self.cache.groups else 0
        room = (held + min(free)) * ps - have if self.cache.groups else n
        return max(0, min(n, room))

    def _preempt(self, r: Request) -> None:
        self.running.remove(r)
        if self.cache.has(r.id):
            self.cache.close(r.id)
        r.computed = 0
        r.state = WAITING
        r.preemptions += 1
        self.counters["preemptions"] += 1
        self.waiting.appendleft(r)

    def _fail(self, r: Request, why: str) -> None:
        if r in self.running:
            self.running.remove(r)
        if self.cache.has(r.id):
            self.cache.close(r.id)
        r.state = FINISHED
        r.finish_reason = "error"
        r.error = why
        self.counters["failed"] += 1

    # ------------------------------------------------------------------ after the step
    def complete(self, plan: StepPlan, sampled: Dict[Any, int]) -> List[Request]:
        """The step ran.  ``sampled`` maps a request id to the token drawn for it (for the
        entries that sample).  Returns the requests that finished; their pages are free."""
        done: List[Request] = []
        for e in plan.entries:
            r = e.request
            if r.state != RUNNING:
                continue        # it ended while this step, planned ahead, was already running
            r.computed += e.count
            if r.output and e.count == 1 and e.samples:
                self.counters["decode_tokens"] += 1
            else:
                self.counters["prompt_tokens"] += e.count
            if not e.samples:
                continue
            tok = int(sampled[r.id])
            r.output.append(tok)
            if tok in self.eos and not r.params.ignore_eos:
                self._finish(r, "stop")            # engine.rs:1185-1188
            elif len(r.output) >= r.params.max_tokens:
                self._finish(r, "length")          # engine.rs:1211-1213
            elif r.sequence_len >= self.max_context:
                self._finish(r, "length")          # engine.rs:1214-1216
            if r.state == FINISHED:
                done.append(r)
        return done

    def _finish(self, r: Request, reason: str) -> None:
        self.running.remove(r)
        if self.cache.has(r.id):
            self.cache.close(r.id)
        r.state = FINISHED
        r.finish_reason = reason
        self.counters["finished"] += 1

    def abort(self, r: Request) -> None:
        """Drop a request wherever it is (a client that went away, engine.rs:695-703)."""
        if r in self.waiting:
            self.waiting.remove(r)
        if r in self.running:
            self.running.remove(r)
        if self.cache.has(r.id):
            self.cache.close(r.id)
        r.state = FINISHED
        r.finish_reason = "aborted"
