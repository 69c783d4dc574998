"""A plain model of the cache bookkeeping, kept beside the tests: pages, block tables per
request, window groups that give pages back, request slots.  The package does this in C++
(``llmario_b200/csrc/host/cache_core.cpp``); the tests drive both with the same random
operations and compare every answer.  Written from the reference's description of its pool and
tables (crates/engine/kv/src/lib.rs:36-176; crates/engine/model/src/kv.rs:402-497, 715-827); it
shares no code with the package."""
from collections import deque
from typing import Any, Deque, Dict, List, Optional, Sequence, Tuple


class PlainFull(Exception):
    def __init__(self, group, needed, free):
        self.group, self.needed, self.free = group, needed, free
        super().__init__(f"group {group}: {needed} needed, {free} free")


class PlainError(RuntimeError):
    pass


class PlainCache:
    """``windows[g]``: keys a query of group g sees (None = all); ``n_pages[g]``: its pool."""

    def __init__(self, n_pages: Sequence[int], windows: Sequence[Optional[int]], page_size: int,
                 max_requests: int, max_context: int, has_state: bool = False):
        self.page_size, self.max_requests, self.max_context = page_size, max_requests, max_context
        self.windows, self.has_state = list(windows), has_state
        self.free: List[Deque[int]] = [deque(range(n)) for n in n_pages]
        self.n_pages = list(n_pages)
        self.requests: Dict[Any, dict] = {}
        self.free_slots: Deque[int] = deque(range(max_requests))
        self.fresh: List[int] = []
        self.updates: List[Dict[Tuple[int, int], int]] = [dict() for _ in n_pages]

    def open(self, rid):
        if rid in self.requests:
            raise PlainError("already open")
        if not self.free_slots:
            raise PlainError("no free slot")
        slot = self.free_slots.popleft()
        self.requests[rid] = dict(slot=slot, length=0, pages=[[] for _ in self.n_pages],
                                  first_live=[0] * len(self.n_pages))
        self.fresh.append(slot)
        return slot

    def _req(self, rid):
        if rid not in self.requests:
            raise PlainError("unknown request")
        return self.requests[rid]

    def _first_needed(self, g, length):
        w = self.windows[g]
        return 0 if w is None else max(0, length - w + 1) // self.page_size

    def pages_needed(self, rid, n):
        r = self._req(rid)
        want = -(-(r["length"] + n) // self.page_size)
        return [max(0, want - len(p)) for p in r["pages"]]

    def reserve(self, growth):
        need = [0] * len(self.n_pages)
        seen = set()
        for rid, n in growth:
            if rid in seen:
                raise PlainError("twice")
            seen.add(rid)
            r = self._req(rid)
            if n <= 0:
                raise PlainError("empty entry")
            if r["length"] + n > self.max_context:
                raise PlainError("context")
            for g, k in enumerate(self.pages_needed(rid, n)):
                need[g] += k
        for g in range(len(self.n_pages)):
            if need[g] > len(self.free[g]):
                raise PlainFull(g, need[g], len(self.free[g]))
        for rid, n in growth:
            r = self._req(rid)
            for g, k in enumerate(self.pages_needed(rid, n)):
                for _ in range(k):
                    p = self.free[g].popleft()
                    self.updates[g][(r["slot"], len(r["pages"][g]))] = p
                    r["pages"][g].append(p)

    def advance(self, rid, n):
        r = self._req(rid)
        if any(r["length"] + n > len(p) * self.page_size for p in r["pages"]):
            raise PlainError("advanced past reserved pages")
        r["length"] += n
        for g in range(len(self.n_pages)):
            keep_from = min(self._first_needed(g, r["length"]), len(r["pages"][g]))
            for j in range(r["first_live"][g], keep_from):
                self.free[g].append(r["pages"][g][j])
                r["pages"][g][j] = -1
                self.updates[g][(r["slot"], j)] = -1
            r["first_live"][g] = max(r["first_live"][g], keep_from)

    def truncate(self, rid, length):
        r = self._req(rid)
        if length > r["length"]:
            raise PlainError("lengthen")
        if self.has_state and length < r["length"]:
            raise PlainError("state")
        for g in range(len(self.n_pages)):
            if self._first_needed(g, length) < r["first_live"][g]:
                raise PlainError("window gone")
        keep = -(-length // self.page_size)
        for g in range(len(self.n_pages)):
            for j in range(keep, len(r["pages"][g])):
                if r["pages"][g][j] >= 0:
                    self.free[g].append(r["pages"][g][j])
                self.updates[g][(r["slot"], j)] = -1
            del r["pages"][g][keep:]
        r["length"] = length

    def close(self, rid):
        r = self._req(rid)
        for g in range(len(self.n_pages)):
            for j, p in enumerate(r["pages"][g]):
                if p >= 0:
                    self.free[g].append(p)
                    self.updates[g][(r["slot"], j)] = -1
        del self.requests[rid]
        self.free_slots.append(r["slot"])
        if r["slot"] in self.fresh:
            self.fresh.remove(r["slot"])

    def take_updates(self):
        out = [sorted((s, j, p) for (s, j), p in u.items()) for u in self.updates]
        self.updates = [dict() for _ in self.n_pages]
        return out

    def take_fresh(self):
        out, self.fresh = self.fresh, []
        return out
