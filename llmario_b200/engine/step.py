"""The step function: one batch of (request, its next tokens) through the model, from the cache.

The contract is the reference's ``forward_batch`` (crates/engine/model/src/forward.rs:204-325):
every entry appends its tokens to its own request at positions ``length ..``; entries may be a
single decoded token or a portion of a prompt, in any mix; a request appears at most once; when
the pages do not suffice the step refuses and changes nothing.  Beyond the reference, the caller
says at which of the step's tokens it wants logits (the reference returns each entry's last).

All tokens of all entries are stacked into one batch of rows; one small array of integers
(token ids, positions, request slots, wanted rows, block-table changes) goes to the device per
step in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from ..cache import CacheError, CacheFull, CacheManager, PagedKV
from ..parts import Segment, StepContext, Workspace
from . import native
from .model import Model


@dataclass
class StepEntry:
    request: Any
    tokens: Sequence[int]
    want: Sequence[int] = ()      # indices into ``tokens`` whose logits are returned


class StepError(ValueError):
    """A batch that breaks the step function's contract."""


def _round4(n: int) -> int:
    return (n + 3) & ~3


HEADER = 16                    # first words of the integer array: block-table changes per group
GRAPH_UPDATES_PER_ROW = 4      # room for block-table changes per row in a recorded step


class ModelRunner:
    """Owns the model, its cache and the per-step device buffers."""

    def __init__(self, model: Model, page_size: int = 64, n_pages: Optional[int] = None,
                 max_requests: int = 64, max_context: Optional[int] = None,
                 token_budget: int = 2048, cache_tokens: Optional[int] = None,
                 use_graphs: bool = True, use_native: bool = True):
        self.model = model
        self.device = model.device
        if self.device.type != "cuda":
            raise RuntimeError("llmario_b200 runs on a CUDA device; there is no CPU path "
                               f"(asked for {self.device})")
        kernels.lib()   # fail now, loudly, if the kernels cannot be built or loaded
        self.page_size = int(page_size)
        self.max_context = int(max_context or model.spec.max_positions)
        self.max_requests = int(max_requests)
        self.token_budget = int(token_budget)
        needs, reads = model.cache_needs()
        if n_pages is None:
            if cache_tokens is not None:
                tokens = int(cache_tokens)
            else:
                # room for every request slot at full context, or what nine tenths of the free
                # device memory hold, whichever is less
                tokens = self.max_requests * self.max_context
                per_token = sum(2 * n.num_kv_heads * n.head_dim for n, r in zip(needs, reads)
                                if isinstance(n, PagedKV) and r is None) * \
                    torch.empty((), dtype=model.dtype).element_size()
                if per_token:
                    free = torch.cuda.mem_get_info(self.device)[0]
                    tokens = max(self.page_size, min(tokens, int(0.9 * free) // per_token))
            n_pages = -(-int(tokens) // self.page_size)
        self.cache = CacheManager(needs, reads, self.page_size, int(n_pages), self.max_requests,
                                  self.max_context)
        self.cache.allocate_storage(model.dtype, self.device)
        self.workspace = Workspace(self.device)
        # blocks that are the standard arrangement of the standard parts are driven from C++,
        # one call per run of them; every other block runs through its own forward()
        self.native = native.NativeLayers(model, self.cache) if use_native else None
        if self.native is not None and not self.native.any():
            self.native = None
        self._meta_dev: Optional[torch.Tensor] = None
        self._meta_host: List[Optional[torch.Tensor]] = [None, None]
        self._meta_event: List[Optional[torch.cuda.Event]] = [None, None]
        self._flip = 0
        self._meta_generation = 0
        # (the header of the step's integer array has a word per cache group and one for the
        # number of fresh request slots)
        self.use_graphs = bool(use_graphs) and len(self.cache.groups) < HEADER and \
            model.graph_safe
        self._graphs: Dict[Any, Any] = {}
        self._graph_seen: Dict[Any, Any] = {}
        self.counters = {"steps": 0, "rows": 0, "max_entries_in_step": 0, "refused_steps": 0,
                         "graphs_recorded": 0, "graph_replays": 0, "failed_launches": 0,
                         "h2d_bytes": 0}
        self._carried_updates: Optional[List[np.ndarray]] = None   # of a step that failed

    # ------------------------------------------------------------------ requests
    def open(self, request: Any) -> None:
        self.cache.open(request)

    def close(self, request: Any) -> None:
        if self.cache.has(request):
            self.cache.close(request)

    def length(self, request: Any) -> int:
        return self.cache.length(request)

    def free_tokens(self) -> int:
        return min(self.cache.free_pages(), default=0) * self.page_size

    # ------------------------------------------------------------------ the step
    def _validate(self, entries: Sequence[StepEntry]) -> int:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        rows = 0
        vocab = self.model.vocab_size
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r}: an entry needs at least one token")
            if min(e.tokens) < 0 or max(e.tokens) >= vocab:
                bad = [t for t in e.tokens if not 0 <= int(t) < vocab][0]
                raise StepError(f"request {e.request!r}: token {bad} outside the vocabulary "
                                f"of {vocab}")
            if e.want and (min(e.want) < 0 or max(e.want) >= n):
                bad = [w for w in e.want if not 0 <= int(w) < n][0]
                raise StepError(f"request {e.request!r}: wanted place {bad} outside its "
                                f"{n} tokens")
            rows += n
        new = [e.request for e in entries if not self.cache.has(e.request)]
        if len(new) > self.cache.free_slots():
            raise StepError(f"{len(new)} new requests but only {self.cache.free_slots()} "
                            f"free request slots (max_requests={self.max_requests})")
        return rows

    def _meta_buffers(self, words: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
        if self._meta_dev is None or self._meta_dev.numel() < words:
            cap = max(4096, 2 * words)
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._meta_host = [torch.empty(cap, dtype=torch.int32, pin_memory=True)
                               for _ in range(2)]
            self._meta_event = [None, None]
            self._meta_generation += 1
        i = self._flip
        self._flip ^= 1
        ev = self._meta_event[i]
        if ev is not None:
            ev.synchronize()
        return self._meta_dev, self._meta_host[i], i

    def step(self, entries: Sequence[StepEntry],
             device_tokens: Optional[Tuple[torch.Tensor, Sequence[int]]] = None) -> torch.Tensor:
        """Run the tokens of ``entries`` as one batch.  Returns float32 logits
        ``[number of wanted places, vocab]`` on the device, in the order of the entries and of
        each entry's ``want``.  Raises :class:`CacheFull` with nothing changed when the pages
        do not suffice.

        ``device_tokens = (source, index)``: row i of the step takes its token from
        ``source[index[i]]`` (int32, on the device) when ``index[i] >= 0``, whatever the entry
        says: the token was drawn by an earlier step and has not been read by the host yet."""
        rows = self._validate(entries)
        if device_tokens is not None and len(device_tokens[1]) != rows:
            raise StepError("device_tokens needs one index for every row of the step")
        cache = self.cache
        opened = []
        try:
            for e in entries:
                if not cache.has(e.request):
                    cache.open(e.request)
                    opened.append(e.request)
            cache.reserve([(e.request, len(e.tokens)) for e in entries])
        except (CacheFull, CacheError):
            for r in opened:
                cache.close(r)
            self.counters["refused_steps"] += 1
            raise

        # ---- one array of integers for the whole step
        segments: List[Segment] = []
        want: List[int] = []
        if rows == len(entries):      # single tokens only: no per-entry array work
            slot, pos = cache.info_many([e.request for e in entries])
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=rows)
            for i, e in enumerate(entries):
                if e.want:
                    want.append(i)
                segments.append(Segment(e.request, int(slot[i]), i, 1, int(pos[i])))
        else:
            tokens = np.empty(rows, dtype=np.int32)
            pos = np.empty(rows, dtype=np.int32)
            slot = np.empty(rows, dtype=np.int32)
            r0 = 0
            for e in entries:
                n = len(e.tokens)
                s, p0 = cache.info(e.request)
                tokens[r0:r0 + n] = np.asarray(e.tokens, dtype=np.int32)
                pos[r0:r0 + n] = np.arange(p0, p0 + n, dtype=np.int32)
                slot[r0:r0 + n] = s
                want += [r0 + int(w) for w in e.want]
                segments.append(Segment(e.request, s, r0, n, p0))
                r0 += n
        updates = self._with_carried(cache.take_table_updates())
        n_want = len(want)
        max_pos = int(pos.max())

        # A step of single tokens has the same launches every time: it is recorded once as a
        # CUDA graph per (rows, wanted rows, context bucket) and replayed.  Its layout of the
        # integer array is fixed, with room for a bounded number of block-table changes.
        graph_key = None
        if self.use_graphs and rows == len(entries) and \
                all(len(u) <= GRAPH_UPDATES_PER_ROW * rows for u in updates):
            bucket = 1 << max(7, max_pos.bit_length())
            graph_key = (rows, n_want, bucket)
        upd_cap = [GRAPH_UPDATES_PER_ROW * rows if graph_key else len(u) for u in updates]

        o_tok = HEADER
        o_pos, o_slot, o_want = o_tok + _round4(rows), o_tok + 2 * _round4(rows), \
            o_tok + 3 * _round4(rows)
        o_upd = []
        off = o_want + _round4(n_want)
        for cap in upd_cap:
            o_upd.append(off)
            off += _round4(3 * cap)
        # request slots opened for this step, whose fixed-size state starts at zero
        fresh = cache.take_fresh_slots() if cache.state else []
        fresh_cap = (rows if graph_key else len(fresh)) if cache.state else 0
        o_fresh = off
        off += _round4(fresh_cap)
        o_src = off                      # behind everything a recorded graph reads
        if device_tokens is not None:
            off += _round4(rows)
        dev, host, which = self._meta_buffers(off)
        h = host.numpy()
        h[:HEADER] = 0
        for gi, u in enumerate(updates):
            h[gi] = len(u)
        h[HEADER - 1] = len(fresh)
        if fresh:
            h[o_fresh:o_fresh + len(fresh)] = np.asarray(fresh, dtype=np.int32)
        h[o_tok:o_tok + rows] = tokens
        h[o_pos:o_pos + rows] = pos
        h[o_slot:o_slot + rows] = slot
        if want:
            h[o_want:o_want + n_want] = np.asarray(want, dtype=np.int32)
        for u, o in zip(updates, o_upd):
            if len(u):
                h[o:o + 3 * len(u)] = u.reshape(-1)
        if device_tokens is not None:
            h[o_src:o_src + rows] = np.asarray(device_tokens[1], dtype=np.int32)
        dev[:off].copy_(host[:off], non_blocking=True)
        self.counters["h2d_bytes"] += 4 * off     # (work items of mixed steps go by the driver)
        if device_tokens is not None:
            kernels.patch_tokens(dev[o_tok:o_tok + rows], device_tokens[0],
                                 dev[o_src:o_src + rows])
        ev = torch.cuda.Event()
        ev.record()
        self._meta_event[which] = ev

        ctx = StepContext(rows=rows, tokens=dev[o_tok:o_tok + rows],
                          row_pos=dev[o_pos:o_pos + rows], row_slot=dev[o_slot:o_slot + rows],
                          segments=segments, dtype=self.model.dtype, device=self.device,
                          workspace=self.workspace, cache=cache, fresh_slots=fresh,
                          max_pos=(graph_key[2] - 1) if graph_key else max_pos)
        want_dev = dev[o_want:o_want + n_want]

        def forward() -> torch.Tensor:
            for gi, (g, o, cap) in enumerate(zip(cache.groups, o_upd, upd_cap)):
                if graph_key:
                    kernels.table_update_counted(g.table, dev[o:o + 3 * cap], dev[gi:gi + 1], cap)
                elif cap:
                    kernels.table_update(g.table, dev[o:o + 3 * cap], cap)
            if fresh_cap:
                for st in cache.state.values():
                    kernels.zero_slots(st, dev[o_fresh:o_fresh + fresh_cap],
                                       dev[HEADER - 1:HEADER], fresh_cap)
            return self._forward(ctx, want_dev, n_want)

        try:
            if graph_key is None:
                logits = forward()
            else:
                logits = self._graph_step(graph_key, forward)
        except BaseException:
            self._after_failed_launch(updates, opened)
            raise
        for e in entries:
            cache.advance(e.request, len(e.tokens))
        c = self.counters
        c["steps"] += 1
        c["rows"] += rows
        c["max_entries_in_step"] = max(c["max_entries_in_step"], len(entries))
        return logits

    def _with_carried(self, updates: List[np.ndarray]) -> List[np.ndarray]:
        """The block-table changes of this step, behind those of an earlier step that failed
        before it could apply them (one triple per cell, the later value wins)."""
        carried, self._carried_updates = self._carried_updates, None
        if carried is None:
            return updates
        out = []
        for old, new in zip(carried, updates):
            cells = {(int(s), int(i)): int(p) for s, i, p in old}
            cells.update({(int(s), int(i)): int(p) for s, i, p in new})
            out.append(np.array([(s, i, p) for (s, i), p in cells.items()],
                                dtype=np.int32).reshape(-1, 3))
        return out

    def _after_failed_launch(self, updates: List[np.ndarray], opened: Sequence[Any]) -> None:
        """A launch of the step raised (a kernel refused a size, a buffer could not grow).  The
        requests have not advanced.  What the step had already taken is put back so that later
        steps are right: its block-table changes are kept for the next step, requests that it
        opened are closed, and every workspace buffer is dropped (a split-K destination that is
        kept at zero may hold partial sums), which also drops the recorded steps."""
        self._carried_updates = updates
        for r in opened:
            if self.cache.has(r):
                self.cache.close(r)
        self.drop_buffers()
        self.counters["failed_launches"] += 1

    def drop_recordings(self) -> None:
        """Forget every recorded step (they are recorded again when their shapes come back)."""
        self._graphs.clear()
        self._graph_seen.clear()

    def drop_buffers(self) -> None:
        """Forget every temporary buffer, those of the native driver included, and with them
        the recorded steps: after a failure a buffer that is kept at zero may hold sums."""
        self.drop_recordings()
        self.workspace.drop()
        if self.native is not None:
            native.arena_drop()

    def _generation(self):
        return (self.workspace.generation, self._meta_generation,
                native.arena_generation() if self.native is not None else 0)

    def _forward(self, ctx: StepContext, want_dev: torch.Tensor, n_want: int) -> torch.Tensor:
        """Embedding, every layer call of the run order, final norm and head at the wanted
        rows.  Returns a view of a workspace buffer: read it before the next step."""
        m = self.model
        x = ctx.buffer("x", (ctx.rows, m.hidden_size), torch.float32)
        m.embedding.forward(ctx, ctx.tokens, x)
        nat = self.native
        if nat is not None:
            nat.begin_step(ctx, x)
        calls, i = m.calls, 0
        while i < len(calls):
            n = nat.runs.get(i) if nat is not None else None
            if n:
                nat.run(i, n)
                i += n
            else:
                m.blocks[calls[i].layer].forward(ctx, calls[i], x)
                i += 1
        logits = ctx.buffer("logits", (n_want, m.vocab_size), torch.float32)
        if n_want:
            hsel = ctx.buffer("head.h", (n_want, m.hidden_size))
            m.final_norm.apply(ctx, x, hsel, want_dev)
            m.head.forward(ctx, hsel, logits)
        return logits

    def _graph_step(self, key, forward) -> torch.Tensor:
        """Run ``forward`` eagerly the first time a key is seen, record it the second time,
        replay the recording from then on.  A recording is dropped when a workspace buffer or
        the integer array has moved since."""
        gen = self._generation()
        rec = self._graphs.get(key)
        if rec is not None and rec[0] == gen:
            rec[1].replay()
            self.counters["graph_replays"] += 1
            kernels.launches += rec[3]       # the kernels of this library inside the recording
            return rec[2]
        if self._graph_seen.get(key) != gen:
            self._graph_seen[key] = gen          # warm: sizes every buffer, loads every kernel
            out = forward()
            if self._generation() != gen:
                self._graph_seen[key] = self._generation()
            return out
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        before = kernels.launches
        with torch.cuda.graph(graph):
            out = forward()
        recorded = kernels.launches - before
        self._graphs[key] = (gen, graph, out, recorded)
        self.counters["graphs_recorded"] += 1
        graph.replay()
        return out
