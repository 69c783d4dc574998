"""Cache manager: pages of keys and values with a block table per request, and slots of
fixed-size state per request.

What the reference does (crates/engine/kv/src/lib.rs:36-176; crates/engine/model/src/kv.rs:
402-497, 715-827): a pool of fixed-size blocks, a table of block ids per sequence (position ->
``table[pos // block]``, slot ``pos % block``), all-or-nothing allocation that refuses with
"needed / free" before changing anything, separate storage classes for layers that keep every
key, layers that keep a window of them, and layers with a fixed-size recurrent state.

Here layers with the same need share a *group*: one pool of pages, one device tensor
``[page][cache slot of the group][K|V][kv head][position in page][head dim]`` and one block
table.  A group whose layers only look back ``window`` keys gives a page back as soon as every
key in it is out of reach of any later query.  Fixed-size state lives in one tensor per
run-order entry, indexed by the request's slot.

All bookkeeping is host-side Python and runs without a GPU; storage is allocated separately by
:meth:`CacheManager.allocate_storage`.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


class CacheFull(Exception):
    """Not enough free pages for a step; nothing was changed (the reference's ``KvFull``,
    kv.rs:554-559)."""

    def __init__(self, group: int, needed: int, free: int):
        self.group, self.needed, self.free = group, needed, free
        super().__init__(f"cache group {group}: {needed} pages needed, {free} free")


class CacheError(RuntimeError):
    """A misuse of the cache manager (unknown request, double free, context overflow)."""


@dataclass(frozen=True)
class PagedKV:
    """A layer that keeps keys and values per token.  ``window``: how many keys a query sees
    (None = all)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """A layer that keeps a state of fixed shape per request."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class PagePool:
    """Page ids 0..n-1.  ``alloc`` is all-or-nothing; a freed page goes to the back of the
    queue, so the page freed longest ago is handed out first (lib.rs:36-128)."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free: Deque[int] = deque(range(n_pages))
        self._held = [False] * n_pages

    @property
    def free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> Optional[List[int]]:
        if n > len(self._free):
            return None
        out = [self._free.popleft() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def release(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages or not self._held[p]:
                raise CacheError(f"page {p} released but not held")
            self._held[p] = False
            self._free.append(p)

    def held(self) -> int:
        return sum(self._held)


@dataclass
class _Group:
    need: PagedKV
    n_pages: int
    entries: List[int] = field(default_factory=list)   # run-order entries stored here
    pool: PagePool = None                               # type: ignore[assignment]
    storage: Optional[torch.Tensor] = None              # [page, slot, 2, Hkv, page_size, hd]
    table: Optional[torch.Tensor] = None                # device int32 [requests, pages/request]
    # (request slot, page index) -> page id, changes not yet sent to the device table
    updates: Dict[Tuple[int, int], int] = field(default_factory=dict)


@dataclass
class CacheView:
    """What a layer call gets: where its keys and values live."""

    k: torch.Tensor          # the group's storage, offset to this call's K plane of page 0
    v: torch.Tensor
    page_stride: int         # elements from one page to the next
    block_table: torch.Tensor
    page_size: int
    group: int
    storage: Optional[torch.Tensor] = None   # the group's whole tensor, for kernels that tile it
    slot: int = 0                            # this call's cache slot inside the group


class _Request:
    __slots__ = ("slot", "length", "pages", "first_live")

    def __init__(self, slot: int, n_groups: int):
        self.slot = slot
        self.length = 0
        self.pages: List[List[int]] = [[] for _ in range(n_groups)]   # -1 = given back
        self.first_live = [0] * n_groups


class CacheManager:
    """``needs[i]`` is what run-order entry ``i`` keeps (PagedKV, FixedState or None);
    ``reads[i]`` names the entry whose cache entry ``i`` reads instead (or None)."""

    def __init__(self, needs: Sequence[Any], reads: Sequence[Optional[int]], page_size: int,
                 n_pages: int, max_requests: int, max_context: int):
        if page_size <= 0 or n_pages <= 0 or max_requests <= 0:
            raise CacheError("page_size, n_pages and max_requests must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_context = max_context
        self.pages_per_request = -(-max_context // page_size)
        self.groups: List[_Group] = []
        self._where: Dict[int, Tuple[int, int]] = {}   # entry -> (group, slot in group)
        self._state_need: Dict[int, FixedState] = {}
        self.state: Dict[int, torch.Tensor] = {}
        by_need: Dict[PagedKV, int] = {}
        for i, need in enumerate(needs):
            if reads[i] is not None:
                continue
            if isinstance(need, PagedKV):
                g = by_need.get(need)
                if g is None:
                    g = len(self.groups)
                    by_need[need] = g
                    self.groups.append(_Group(need, n_pages, pool=PagePool(n_pages)))
                self._where[i] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(i)
            elif isinstance(need, FixedState):
                self._state_need[i] = need
            elif need is not None:
                raise CacheError(f"run-order entry {i}: unknown cache need {need!r}")
        for i, src in enumerate(reads):
            if src is not None:
                if src in self._where:
                    self._where[i] = self._where[src]
                elif src in self._state_need:
                    raise CacheError(f"entry {i} cannot read the fixed-size state of {src}")
                else:
                    raise CacheError(f"entry {i} reads the cache of {src}, which has none")
        self._requests: Dict[Any, _Request] = {}
        self._free_slots: Deque[int] = deque(range(max_requests))
        self._fresh_slots: List[int] = []      # slots whose state must be zeroed before use
        self.device: Optional[torch.device] = None
        self.dtype: Optional[torch.dtype] = None
        self.counters = {"pages_allocated": 0, "pages_released": 0, "window_releases": 0,
                         "refusals": 0}

    # ------------------------------------------------------------------ storage
    def allocate_storage(self, dtype: torch.dtype, device) -> None:
        self.device, self.dtype = torch.device(device), dtype
        for g in self.groups:
            n = g.need
            # per KV head the positions of a page lie one after the other: a kernel that serves
            # one KV head reads page_size * head_dim contiguous elements per page
            g.storage = torch.zeros((g.n_pages, len(g.entries), 2, n.num_kv_heads,
                                     self.page_size, n.head_dim), dtype=dtype, device=device)
            g.table = torch.full((self.max_requests, self.pages_per_request), -1,
                                 dtype=torch.int32, device=device)
        for i, need in self._state_need.items():
            self.state[i] = torch.zeros((self.max_requests, *need.shape), dtype=need.dtype,
                                        device=device)

    def storage_bytes(self, dtype: torch.dtype) -> int:
        size = torch.empty((), dtype=dtype).element_size()
        total = 0
        for g in self.groups:
            total += (g.n_pages * len(g.entries) * 2 * self.page_size * g.need.num_kv_heads *
                      g.need.head_dim * size)
        return total

    def view(self, entry: int) -> Optional[CacheView]:
        if entry not in self._where:
            return None
        gi, slot = self._where[entry]
        g = self.groups[gi]
        st = g.storage
        return CacheView(st[0, slot, 0], st[0, slot, 1], st.stride(0), g.table, self.page_size,
                         gi, st, slot)

    def state_of(self, entry: int) -> Optional[torch.Tensor]:
        return self.state.get(entry)

    # ------------------------------------------------------------------ requests
    def open(self, request_id: Any) -> int:
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already open")
        if not self._free_slots:
            raise CacheError("no free request slot")
        slot = self._free_slots.popleft()
        self._requests[request_id] = _Request(slot, len(self.groups))
        self._fresh_slots.append(slot)
        return slot

    def has(self, request_id: Any) -> bool:
        return request_id in self._requests

    def slot(self, request_id: Any) -> int:
        return self._req(request_id).slot

    def length(self, request_id: Any) -> int:
        return self._req(request_id).length

    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self) -> List[int]:
        return [g.pool.free for g in self.groups]

    def live_requests(self) -> List[Any]:
        return list(self._requests)

    def _req(self, request_id: Any) -> _Request:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheError(f"unknown request {request_id!r}") from None

    def _first_needed_page(self, g: _Group, length: int) -> int:
        """First page that a query at position >= length can still reach."""
        w = g.need.window
        if w is None:
            return 0
        return max(0, length - w + 1) // self.page_size

    def pages_needed(self, request_id: Any, new_tokens: int) -> List[int]:
        """Pages each group must add so that the request can grow by ``new_tokens``."""
        r = self._req(request_id)
        new_len = r.length + new_tokens
        want = -(-new_len // self.page_size)
        return [max(0, want - len(r.pages[gi])) for gi in range(len(self.groups))]

    def reserve(self, growth: Sequence[Tuple[Any, int]]) -> None:
        """Make room for every (request, new tokens) of a step, or change nothing and raise
        :class:`CacheFull` (crates/engine/model/src/forward.rs:245-259)."""
        need = [0] * len(self.groups)
        seen = set()
        for rid, n in growth:
            if rid in seen:
                raise CacheError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            r = self._req(rid)
            if n <= 0:
                raise CacheError(f"request {rid!r}: a step entry needs at least one token")
            if r.length + n > self.max_context:
                raise CacheError(f"request {rid!r}: {r.length} + {n} tokens exceed the context "
                                 f"of {self.max_context}")
            for gi, k in enumerate(self.pages_needed(rid, n)):
                need[gi] += k
        for gi, g in enumerate(self.groups):
            if need[gi] > g.pool.free:
                self.counters["refusals"] += 1
                raise CacheFull(gi, need[gi], g.pool.free)
        if not any(need):
            return
        for rid, n in growth:
            r = self._req(rid)
            for gi, k in enumerate(self.pages_needed(rid, n)):
                if k == 0:
                    continue
                g = self.groups[gi]
                pages = g.pool.alloc(k)
                assert pages is not None
                self.counters["pages_allocated"] += k
                for p in pages:
                    g.updates[(r.slot, len(r.pages[gi]))] = p
                    r.pages[gi].append(p)

    def advance(self, request_id: Any, n: int) -> None:
        """The request now holds ``n`` more tokens; pages that a window has passed go back."""
        r = self._req(request_id)
        r.length += n
        for gi in range(len(self.groups)):
            if r.length > len(r.pages[gi]) * self.page_size:
                raise CacheError(f"request {request_id!r} advanced past its reserved pages")
        for gi, g in enumerate(self.groups):
            keep_from = min(self._first_needed_page(g, r.length), len(r.pages[gi]))
            if keep_from > r.first_live[gi]:
                gone = r.pages[gi][r.first_live[gi]:keep_from]
                g.pool.release(gone)
                self.counters["pages_released"] += len(gone)
                self.counters["window_releases"] += len(gone)
                for j in range(r.first_live[gi], keep_from):
                    r.pages[gi][j] = -1
                    g.updates[(r.slot, j)] = -1
                r.first_live[gi] = keep_from

    def truncate(self, request_id: Any, length: int) -> None:
        """Forget everything past ``length`` tokens (kv.rs:792-816).  A group that has given
        pages back to its window cannot be rewound into them."""
        r = self._req(request_id)
        if length > r.length:
            raise CacheError("truncate cannot lengthen a request")
        if self._state_need and length < r.length:
            raise CacheError("a request with fixed-size state cannot be rewound; close it")
        keep = -(-length // self.page_size)
        for gi, g in enumerate(self.groups):
            if self._first_needed_page(g, length) < r.first_live[gi]:
                raise CacheError(f"group {gi}: the window has already given back pages that a "
                                 f"request of {length} tokens needs")
            gone = [p for p in r.pages[gi][keep:] if p >= 0]
            g.pool.release(gone)
            self.counters["pages_released"] += len(gone)
            for j in range(keep, len(r.pages[gi])):
                g.updates[(r.slot, j)] = -1
            del r.pages[gi][keep:]
        r.length = length

    def close(self, request_id: Any) -> None:
        """The request is over: its pages, its slot and its state go back."""
        r = self._req(request_id)
        for gi, g in enumerate(self.groups):
            gone = [p for p in r.pages[gi] if p >= 0]
            g.pool.release(gone)
            self.counters["pages_released"] += len(gone)
            for j, p in enumerate(r.pages[gi]):
                if p >= 0:
                    g.updates[(r.slot, j)] = -1
        del self._requests[request_id]
        self._free_slots.append(r.slot)
        if r.slot in self._fresh_slots:
            self._fresh_slots.remove(r.slot)

    # ------------------------------------------------------------------ device mirror
    def take_table_updates(self) -> List[np.ndarray]:
        """Per group, the (request slot, page index, page id) triples since the last call; one
        triple per table cell (the last value wins), so they may be applied in any order."""
        out = []
        for g in self.groups:
            out.append(np.asarray([(s, j, p) for (s, j), p in g.updates.items()],
                                  dtype=np.int32).reshape(-1, 3))
            g.updates = {}
        return out

    def take_fresh_slots(self) -> List[int]:
        out, self._fresh_slots = self._fresh_slots, []
        return out

    def pages_of(self, request_id: Any, group: int = 0) -> List[int]:
        return list(self._req(request_id).pages[group])

    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held."""
        for gi, g in enumerate(self.groups):
            held: List[int] = []
            for r in self._requests.values():
                held += [p for p in r.pages[gi] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {gi}: a page is held twice")
            free = list(g.pool._free)
            if set(free) & set(held):
                raise CacheError(f"group {gi}: a page is both free and held")
            if len(free) != len(set(free)):
                raise CacheError(f"group {gi}: a page is in the free queue twice")
            if len(free) + len(held) != g.n_pages:
                raise CacheError(f"group {gi}: {g.n_pages - len(free) - len(held)} pages lost")
            if g.pool.held() != len(held):
                raise CacheError(f"group {gi}: the pool's own count of held pages is off")
        slots = [r.slot for r in self._requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots):
            raise CacheError("a request slot is held twice or both free and held")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a request slot was lost")
