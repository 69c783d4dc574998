"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.  The decisions are made in native code
(``llmario_b200/csrc/host/sched_core.cpp``, in the same library as the cache bookkeeping, which
it asks directly); this module holds what the native side has no use for, the requests' token
ids and sampling parameters, and mirrors its queues as Python objects.

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

import ctypes
import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Sequence

from ..cache import CacheManager
from ..csrc.build import load_host_library
from ..sampling import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
_REASONS = {1: "stop", 2: "length", 3: "error", 4: "aborted"}
_COUNTERS = ("admitted", "finished", "preemptions", "failed", "steps_planned", "prompt_tokens",
             "decode_tokens", "steps_planned_ahead")
_TOO_LARGE = "KV cache full: the request does not fit the cache even alone"


@dataclass
class Request:
    id: Any
    prompt: List[int]
    params: SamplingParams
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


_declared = False


def _native():
    """The host library with the scheduler's functions declared."""
    global _declared
    lib = load_host_library()
    if not _declared:
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        sigs = {
            "llm_sched_new": ([P, I, I, I, I], P),
            "llm_sched_delete": ([P], None),
            "llm_sched_set_eos": ([P, I, P], None),
            "llm_sched_add": ([P, L, I, I, I, I], I),
            "llm_sched_forget": ([P, L], I),
            "llm_sched_has_work": ([P], I),
            "llm_sched_request": ([P, L, P], I),
            "llm_sched_plan": ([P, I, P, P, P, P], I),
            "llm_sched_plan_ahead": ([P, I, P, P, I, I, P, P, P, P], I),
            "llm_sched_complete": ([P, I, P, P, P, P, P], I),
            "llm_sched_abort": ([P, L], I),
            "llm_sched_fail": ([P, L], I),
            "llm_sched_queues": ([P, I, P, P, P], I),
            "llm_sched_counters": ([P, P], None),
        }
        for name, (args, res) in sigs.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, res
        _declared = True
    return lib


class Scheduler:
    def __init__(self, cache: CacheManager, token_budget: int = 512, max_context: Optional[int]
                 = None, eos_token_ids: Sequence[int] = ()):
        if token_budget <= 0:
            raise ValueError("token_budget must be positive")
        self.cache = cache
        self.token_budget = int(token_budget)
        self.max_context = int(max_context or cache.max_context)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []      # in order of admission
        self._arrivals = itertools.count()
        self._lib = _native()
        self._s = self._lib.llm_sched_new(cache.core, len(cache.groups), cache.page_size,
                                          self.token_budget, self.max_context)
        if not self._s:
            raise ValueError("the native scheduler refused these sizes")
        self.eos = eos_token_ids
        self._by_key: Dict[int, Request] = {}
        self._cap = 0
        self._room(64)

    def __del__(self):
        if getattr(self, "_s", None) and getattr(self, "_lib", None) is not None:
            self._lib.llm_sched_delete(self._s)
            self._s = None

    def _room(self, n: int) -> None:
        """Arrays for plans and events of up to ``n`` requests."""
        if n <= self._cap:
            return
        cap = max(64, 2 * n)
        self._keys = (ctypes.c_int64 * cap)()
        self._triples = (ctypes.c_int * (3 * cap))()
        self._events = (ctypes.c_int64 * cap)()
        self._in_keys = (ctypes.c_int64 * cap)()
        self._in_triples = (ctypes.c_int * (3 * cap))()
        self._tokens = (ctypes.c_int * cap)()
        self._reasons = (ctypes.c_int * cap)()
        self._n_events = (ctypes.c_int * 3)()
        self._cap = cap

    @property
    def eos(self) -> frozenset:
        """The token ids that end a request (unless it asks to ignore them)."""
        return self._eos

    @eos.setter
    def eos(self, token_ids) -> None:
        self._eos = frozenset(int(e) for e in token_ids)
        arr = (ctypes.c_int * max(1, len(self._eos)))(*sorted(self._eos))
        self._lib.llm_sched_set_eos(self._s, len(self._eos), arr)

    @property
    def counters(self) -> Dict[str, int]:
        out = (ctypes.c_longlong * len(_COUNTERS))()
        self._lib.llm_sched_counters(self._s, out)
        return dict(zip(_COUNTERS, out))

    # ------------------------------------------------------------------ queue
    def add(self, request: Request) -> None:
        """Queue a request.  An empty prompt, or one that leaves no room in the context, is
        refused (engine.rs:788-798)."""
        if not request.prompt:
            raise ValueError("empty prompt")
        if len(request.prompt) >= self.max_context:
            raise ValueError(f"prompt of {len(request.prompt)} tokens does not fit the context "
                             f"of {self.max_context}")
        key = self.cache.name(request.id)
        p = request.params
        rc = self._lib.llm_sched_add(self._s, key, len(request.prompt), int(p.max_tokens),
                                     int(bool(p.ignore_eos)), int(bool(p.penalties_active)))
        if rc != 0:
            raise ValueError(f"request {request.id!r}: the native scheduler answered {rc}")
        request.arrival = next(self._arrivals)
        request.state = WAITING
        self._by_key[key] = request
        self.waiting.append(request)
        self._room(len(self._by_key))

    def has_work(self) -> bool:
        return bool(self._lib.llm_sched_has_work(self._s))

    def _mirror_queues(self) -> None:
        nw, nr = ctypes.c_int(), ctypes.c_int()
        n = self._lib.llm_sched_queues(self._s, self._cap, self._keys, ctypes.byref(nw),
                                       ctypes.byref(nr))
        if n < 0:
            raise RuntimeError("the scheduler's arrays are too small for its queues")
        self.waiting = deque(self._by_key[self._keys[i]] for i in range(nw.value))
        self.running = [self._by_key[self._keys[i]] for i in range(nw.value, n)]

    def _gone(self, r: Request, reason: str, error: Optional[str] = None) -> None:
        """The native side has ended this request and closed it in the cache core."""
        r.state = FINISHED
        r.finish_reason = reason
        r.error = error
        key = self.cache.name(r.id)
        self.cache.closed_in_core(r.id)
        self.cache.unname(r.id)
        self._by_key.pop(key, None)
        self._lib.llm_sched_forget(self._s, key)

    # ------------------------------------------------------------------ planning
    def plan(self) -> StepPlan:
        """Decide the next step.  Changes the queues (admission, preemption, failure) but feeds
        nothing: the caller runs the step and reports back with :meth:`complete`."""
        n = self._lib.llm_sched_plan(self._s, self._cap, self._keys, self._triples, self._events,
                                     self._n_events)
        if n < 0:
            raise RuntimeError(f"the native scheduler answered {n}")
        plan = StepPlan()
        n_pre, n_fail, n_adm = self._n_events
        at = 0
        for _ in range(n_pre):
            r = self._by_key[self._events[at]]
            at += 1
            r.computed = 0
            r.state = WAITING
            r.preemptions += 1
            self.cache.closed_in_core(r.id)
            plan.preempted.append(r)
        failed = [self._by_key[self._events[at + i]] for i in range(n_fail)]
        at += n_fail
        for i in range(n_adm):
            self._by_key[self._events[at + i]].state = RUNNING
        t = self._triples
        plan.entries = [PlanEntry(self._by_key[self._keys[i]], t[3 * i], t[3 * i + 1],
                                  bool(t[3 * i + 2])) for i in range(n)]
        for r in failed:
            self._gone(r, "error", _TOO_LARGE)
            plan.failed.append(r)
        self._mirror_queues()
        return plan

    def plan_ahead(self, flying: StepPlan) -> Optional[StepPlan]:
        """The step after ``flying``, decided while ``flying`` is still running and the tokens it
        draws are unknown, or None when that step cannot be known yet.  The planner runs as for
        any step, on the requests as they will stand when ``flying`` ends without an
        end-of-sequence token: decoding requests get one more token (the one in flight is their
        input), prompts their next portions, waiting requests are admitted into free slots.  A
        request whose last token is in flight (``max_tokens`` or the context reached) is left
        out; it keeps its slot and pages until ``flying`` is reported.  None when ``flying``
        preempted or failed someone, when pages are so short that a request would have to give
        way (that is decided with all facts known), or when nothing could run.  A request that
        does end on an end-of-sequence token drawn by ``flying`` has a row too many in the step
        ahead; :meth:`complete` passes over it.  The cache lengths already count ``flying``."""
        n = len(flying.entries)
        if n == 0 or n > self._cap:
            return None
        for i, e in enumerate(flying.entries):
            self._in_keys[i] = self.cache.name(e.request.id) if e.request.state != FINISHED else 0
            self._in_triples[3 * i] = e.start
            self._in_triples[3 * i + 1] = e.count
            self._in_triples[3 * i + 2] = int(e.samples)
        m = self._lib.llm_sched_plan_ahead(self._s, n, self._in_keys, self._in_triples,
                                           len(flying.preempted) + len(flying.failed), self._cap,
                                           self._keys, self._triples, self._events, self._n_events)
        if m == -1:
            return None
        if m < 0:
            raise RuntimeError(f"the native scheduler answered {m}")
        plan = StepPlan()
        for i in range(self._n_events[2]):
            self._by_key[self._events[i]].state = RUNNING
        t = self._triples
        plan.entries = [PlanEntry(self._by_key[self._keys[i]], t[3 * i], t[3 * i + 1],
                                  bool(t[3 * i + 2])) for i in range(m)]
        if self._n_events[2]:
            self._mirror_queues()
        return plan

    # ------------------------------------------------------------------ after the step
    def complete(self, plan: StepPlan, sampled: Dict[Any, int]) -> List[Request]:
        """The step ran.  ``sampled`` maps a request id to the token drawn for it (for the
        entries that sample).  Returns the requests that finished; their pages are free."""
        entries = [e for e in plan.entries if e.request.state == RUNNING]
        # (a request that is no longer running ended while this step, planned ahead, was
        # already running: it is passed over)
        n = len(entries)
        self._room(n)
        for i, e in enumerate(entries):
            r = e.request
            self._in_keys[i] = self.cache.name(r.id)
            self._in_triples[3 * i] = e.start
            self._in_triples[3 * i + 1] = e.count
            self._in_triples[3 * i + 2] = int(e.samples)
            self._tokens[i] = int(sampled[r.id]) if e.samples else -1
        k = self._lib.llm_sched_complete(self._s, n, self._in_keys, self._in_triples, self._tokens,
                                         self._keys, self._reasons)
        for i, e in enumerate(entries):
            r = e.request
            r.computed += e.count
            if e.samples:
                r.output.append(self._tokens[i])
        done = []
        for i in range(k):
            r = self._by_key[self._keys[i]]
            self._gone(r, _REASONS[self._reasons[i]])
            done.append(r)
        if k:
            self._mirror_queues()
        return done

    def abort(self, r: Request) -> None:
        """Drop a request wherever it is (a client that went away, engine.rs:695-703)."""
        if r.state == FINISHED:
            return
        self._lib.llm_sched_abort(self._s, self.cache.name(r.id))
        self._gone(r, "aborted")
        self._mirror_queues()

    def fail(self, r: Request, error: str) -> None:
        """End a request with ``finish_reason == "error"``: a step it was part of failed on the
        device (the reference's ``Event::Error``, engine.rs:1140).  Its pages are given back."""
        if r.state == FINISHED:
            return
        self._lib.llm_sched_fail(self._s, self.cache.name(r.id))
        self._gone(r, "error", error)
        self._mirror_queues()
