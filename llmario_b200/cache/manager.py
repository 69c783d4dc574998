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

The bookkeeping itself (free pages, the pages of every request, what a window has passed, which
table cells have changed) is C++ (``csrc/host/cache_core.cpp``, compiled by the system's C++
compiler on first use, no GPU needed); this module owns the device tensors, names requests by
whatever hashable id the caller uses, and turns the core's codes into exceptions.  Storage is
allocated separately by :meth:`CacheManager.allocate_storage`.
"""
from __future__ import annotations

import ctypes
import itertools
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..csrc.build import load_host_library


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


_lib = None


def _core():
    """The host library with its functions declared."""
    global _lib
    if _lib is None:
        l = load_host_library()
        P, I, K = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        IP = ctypes.POINTER(ctypes.c_int)
        sigs = {
            "llm_cache_new": (P, [I, IP, IP, I, I, I, I]),
            "llm_cache_delete": (None, [P]),
            "llm_cache_open": (I, [P, K]),
            "llm_cache_has": (I, [P, K]),
            "llm_cache_info": (I, [P, K, IP, IP]),
            "llm_cache_info_many": (I, [P, I, P, P, P]),
            "llm_cache_free_slots": (I, [P]),
            "llm_cache_free_pages": (None, [P, IP]),
            "llm_cache_pages_needed": (I, [P, K, I, IP]),
            "llm_cache_reserve": (I, [P, I, P, P, IP]),
            "llm_cache_advance": (I, [P, K, I]),
            "llm_cache_truncate": (I, [P, K, I, IP]),
            "llm_cache_close": (I, [P, K]),
            "llm_cache_pending_updates": (I, [P, I]),
            "llm_cache_take_updates": (I, [P, I, P]),
            "llm_cache_take_fresh": (I, [P, IP, I]),
            "llm_cache_pages_of": (I, [P, K, I, IP, I]),
            "llm_cache_live": (I, [P, P, I]),
            "llm_cache_counters": (None, [P, P]),
            "llm_cache_check": (I, [P, IP]),
            "llm_pool_new": (P, [I]),
            "llm_pool_delete": (None, [P]),
            "llm_pool_free": (I, [P]),
            "llm_pool_held": (I, [P]),
            "llm_pool_alloc": (I, [P, I, IP]),
            "llm_pool_release": (I, [P, IP, I]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


# what the core's negative codes mean (csrc/host/cache_core.cpp)
_E_UNKNOWN, _E_OPEN_TWICE, _E_NO_SLOT, _E_TWICE, _E_EMPTY, _E_CONTEXT = -1, -2, -3, -4, -5, -6
_E_PAST, _E_LENGTHEN, _E_STATE, _E_WINDOW, _E_NOT_HELD = -7, -8, -9, -10, -11
_CHECK = {-20: "a page is held twice", -21: "a page is both free and held",
          -22: "a page is in the free queue twice", -23: "pages lost",
          -24: "the pool's own count of held pages is off",
          -25: "a request slot is held twice or both free and held",
          -26: "a request slot was lost"}


class PagePool:
    """Page ids 0..n-1.  ``alloc`` is all-or-nothing; a freed page goes to the back of the
    queue, so the page freed longest ago is handed out first (lib.rs:36-128)."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._p = _core().llm_pool_new(n_pages)
        if not self._p:
            raise CacheError("a pool needs at least one page")

    def __del__(self):
        if getattr(self, "_p", None) and _lib is not None:
            _lib.llm_pool_delete(self._p)
            self._p = None

    @property
    def free(self) -> int:
        return _core().llm_pool_free(self._p)

    def alloc(self, n: int) -> Optional[List[int]]:
        out = (ctypes.c_int * max(n, 1))()
        if _core().llm_pool_alloc(self._p, n, out) < 0:
            return None
        return list(out[:n])

    def release(self, pages: Sequence[int]) -> None:
        arr = (ctypes.c_int * max(len(pages), 1))(*pages)
        if _core().llm_pool_release(self._p, arr, len(pages)) != 0:
            raise CacheError(f"a page of {list(pages)} released but not held")

    def held(self) -> int:
        return _core().llm_pool_held(self._p)


@dataclass
class _Group:
    need: PagedKV
    n_pages: int
    entries: List[int] = field(default_factory=list)   # run-order entries stored here
    storage: Optional[torch.Tensor] = None              # [page, slot, 2, Hkv, page_size, hd]
    table: Optional[torch.Tensor] = None                # device int32 [requests, pages/request]


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
                    self.groups.append(_Group(need, n_pages))
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
        G = len(self.groups)
        self._lib = _core()
        pages = (ctypes.c_int * max(G, 1))(*[g.n_pages for g in self.groups])
        windows = (ctypes.c_int * max(G, 1))(*[g.need.window or 0 for g in self.groups])
        self._c = self._lib.llm_cache_new(G, pages, windows, page_size, max_requests, max_context,
                                          int(bool(self._state_need)))
        if not self._c:
            raise CacheError("the cache core refused these sizes")
        self._keys: Dict[Any, int] = {}            # open requests: id -> the core's 64-bit key
        self._ids: Dict[int, Any] = {}
        self._names: Dict[Any, int] = {}           # keys promised before a request is opened
        self._next_key = itertools.count(1)
        self._info = (ctypes.c_int * 4)()
        self._per_group = (ctypes.c_int * max(G, 1))()
        self.device: Optional[torch.device] = None
        self.dtype: Optional[torch.dtype] = None

    def __del__(self):
        if getattr(self, "_c", None) and getattr(self, "_lib", None) is not None:
            self._lib.llm_cache_delete(self._c)
            self._c = None

    @property
    def counters(self) -> Dict[str, int]:
        out = (ctypes.c_longlong * 4)()
        self._lib.llm_cache_counters(self._c, out)
        return {"pages_allocated": out[0], "pages_released": out[1], "window_releases": out[2],
                "refusals": out[3]}

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
    def _key(self, request_id: Any) -> int:
        try:
            return self._keys[request_id]
        except KeyError:
            raise CacheError(f"unknown request {request_id!r}") from None

    def name(self, request_id: Any) -> int:
        """The 64-bit key under which the core will know this request whenever it is open, now
        or later (a request that loses its pages and is opened again keeps it), until
        :meth:`unname`.  The native scheduler asks the core about requests by these keys."""
        key = self._names.get(request_id)
        if key is None:
            key = self._keys.get(request_id)
            if key is None:
                key = next(self._next_key)
            self._names[request_id] = key
        return key

    def unname(self, request_id: Any) -> None:
        self._names.pop(request_id, None)

    @property
    def core(self):
        """The native core's handle (for the native scheduler, which lives in the same library)."""
        return self._c

    def closed_in_core(self, request_id: Any) -> None:
        """The native scheduler has closed this request in the core (preempted, failed or
        finished it): forget it here as well."""
        key = self._keys.pop(request_id, None)
        if key is not None:
            self._ids.pop(key, None)

    def open(self, request_id: Any) -> int:
        if request_id in self._keys:
            raise CacheError(f"request {request_id!r} is already open")
        key = self._names.get(request_id)
        if key is None:
            key = next(self._next_key)
        slot = self._lib.llm_cache_open(self._c, key)
        if slot == _E_NO_SLOT:
            raise CacheError("no free request slot")
        if slot < 0:
            raise CacheError(f"request {request_id!r}: the cache core answered {slot}")
        self._keys[request_id] = key
        self._ids[key] = request_id
        return slot

    def has(self, request_id: Any) -> bool:
        return request_id in self._keys

    def info(self, request_id: Any) -> Tuple[int, int]:
        """(request slot, tokens held)."""
        s, n = ctypes.c_int(), ctypes.c_int()
        if self._lib.llm_cache_info(self._c, self._key(request_id), s, n) != 0:
            raise CacheError(f"unknown request {request_id!r}")
        return s.value, n.value

    def info_many(self, request_ids: Sequence[Any]) -> Tuple[np.ndarray, np.ndarray]:
        """Request slots and lengths of several requests as int32 arrays."""
        n = len(request_ids)
        keys = np.fromiter((self._key(r) for r in request_ids), dtype=np.int64, count=n)
        slots, lengths = np.empty(n, dtype=np.int32), np.empty(n, dtype=np.int32)
        rc = self._lib.llm_cache_info_many(self._c, n, keys.ctypes.data, slots.ctypes.data,
                                           lengths.ctypes.data)
        if rc != 0:
            raise CacheError(f"unknown request {request_ids[-rc - 100]!r}")
        return slots, lengths

    def slot(self, request_id: Any) -> int:
        return self.info(request_id)[0]

    def length(self, request_id: Any) -> int:
        return self.info(request_id)[1]

    def free_slots(self) -> int:
        return self._lib.llm_cache_free_slots(self._c)

    def free_pages(self) -> List[int]:
        self._lib.llm_cache_free_pages(self._c, self._per_group)
        return list(self._per_group[:len(self.groups)])

    def live_requests(self) -> List[Any]:
        return list(self._keys)

    def pages_needed(self, request_id: Any, new_tokens: int) -> List[int]:
        """Pages each group must add so that the request can grow by ``new_tokens``."""
        self._lib.llm_cache_pages_needed(self._c, self._key(request_id), new_tokens,
                                         self._per_group)
        return list(self._per_group[:len(self.groups)])

    def reserve(self, growth: Sequence[Tuple[Any, int]]) -> None:
        """Make room for every (request, new tokens) of a step, or change nothing and raise
        :class:`CacheFull` (crates/engine/model/src/forward.rs:245-259)."""
        n = len(growth)
        seen = set()
        for rid, _ in growth:
            if rid in seen:
                raise CacheError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
        keys = np.fromiter((self._key(rid) for rid, _ in growth), dtype=np.int64, count=n)
        counts = np.fromiter((k for _, k in growth), dtype=np.int32, count=n)
        rc = self._lib.llm_cache_reserve(self._c, n, keys.ctypes.data, counts.ctypes.data,
                                         self._info)
        if rc == 0:
            return
        i = self._info
        if rc == 1:
            raise CacheFull(i[0], i[1], i[2])
        rid = growth[i[0]][0] if 0 <= i[0] < n else None
        if rc == _E_EMPTY:
            raise CacheError(f"request {rid!r}: a step entry needs at least one token")
        if rc == _E_CONTEXT:
            raise CacheError(f"request {rid!r}: {i[1]} + {i[2]} tokens exceed the context of "
                             f"{self.max_context}")
        if rc == _E_TWICE:
            raise CacheError(f"request {rid!r} appears twice in one step")
        raise CacheError(f"request {rid!r}: the cache core answered {rc}")

    def advance(self, request_id: Any, n: int) -> None:
        """The request now holds ``n`` more tokens; pages that a window has passed go back."""
        rc = self._lib.llm_cache_advance(self._c, self._key(request_id), n)
        if rc == _E_PAST:
            raise CacheError(f"request {request_id!r} advanced past its reserved pages")
        if rc != 0:
            raise CacheError(f"request {request_id!r}: the cache core answered {rc}")

    def truncate(self, request_id: Any, length: int) -> None:
        """Forget everything past ``length`` tokens (kv.rs:792-816).  A group that has given
        pages back to its window cannot be rewound into them."""
        rc = self._lib.llm_cache_truncate(self._c, self._key(request_id), length, self._info)
        if rc == 0:
            return
        if rc == _E_LENGTHEN:
            raise CacheError("truncate cannot lengthen a request")
        if rc == _E_STATE:
            raise CacheError("a request with fixed-size state cannot be rewound; close it")
        if rc == _E_WINDOW:
            raise CacheError(f"group {self._info[0]}: the window has already given back pages "
                             f"that a request of {length} tokens needs")
        raise CacheError(f"request {request_id!r}: the cache core answered {rc}")

    def close(self, request_id: Any) -> None:
        """The request is over: its pages, its slot and its state go back."""
        key = self._key(request_id)
        rc = self._lib.llm_cache_close(self._c, key)
        if rc != 0:
            raise CacheError(f"request {request_id!r}: the cache core answered {rc}")
        del self._keys[request_id]
        del self._ids[key]

    # ------------------------------------------------------------------ device mirror
    def take_table_updates(self) -> List[np.ndarray]:
        """Per group, the (request slot, page index, page id) triples since the last call; one
        triple per table cell (the last value wins), so they may be applied in any order."""
        out = []
        for gi in range(len(self.groups)):
            n = self._lib.llm_cache_pending_updates(self._c, gi)
            arr = np.empty((n, 3), dtype=np.int32)
            if n:
                self._lib.llm_cache_take_updates(self._c, gi, arr.ctypes.data)
            out.append(arr)
        return out

    def take_fresh_slots(self) -> List[int]:
        buf = (ctypes.c_int * self.max_requests)()
        n = self._lib.llm_cache_take_fresh(self._c, buf, self.max_requests)
        return list(buf[:n])

    def pages_of(self, request_id: Any, group: int = 0) -> List[int]:
        buf = (ctypes.c_int * self.pages_per_request)()
        n = self._lib.llm_cache_pages_of(self._c, self._key(request_id), group, buf,
                                         self.pages_per_request)
        if n < 0:
            raise CacheError(f"request {request_id!r}, group {group}: the cache core answered {n}")
        return list(buf[:n])

    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held."""
        rc = self._lib.llm_cache_check(self._c, self._info)
        if rc != 0:
            where = f"group {self._info[0]}: " if rc > -25 else ""
            raise CacheError(where + _CHECK.get(rc, f"the cache core answered {rc}"))
        if len(self._keys) + self.free_slots() != self.max_requests:
            raise CacheError("a request slot was lost")
