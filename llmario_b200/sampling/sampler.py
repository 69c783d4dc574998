"""The sampler: per-request state on the host (options, random stream, penalty window) and the
chain itself on the device (``csrc/sampling.cu``).

Order of the chain (crates/engine/decode/src/sampler.rs:234-362): penalties -> greedy? ->
top-k -> top-p -> min-p -> temperature -> softmax -> draw.  The window holds the last
``repeat_last_n`` tokens, prompt included (sampler.rs:374-386).
"""
from __future__ import annotations

import itertools
import os
from collections import deque
from typing import Deque, Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams
from .rng import Xoshiro256StarStar


_serials = itertools.count(1)


class RequestSampler:
    """Sampling state of one request."""

    def __init__(self, params: SamplingParams, vocab_size: int):
        self.serial = next(_serials)      # never repeats: names this object in cached option rows
        self.params = params
        self.vocab_size = vocab_size
        self.seed = params.seed if params.seed is not None else \
            int.from_bytes(os.urandom(8), "little")
        self.rng = Xoshiro256StarStar(self.seed)
        self.window: Deque[int] = deque()
        self.counts: Dict[int, int] = {}

    def accept(self, token: int) -> None:
        """A prompt or generated token enters the penalty window."""
        n = self.params.repeat_last_n
        if n <= 0 or not 0 <= token < self.vocab_size:
            return
        if len(self.window) >= n:
            old = self.window.popleft()
            c = self.counts[old] - 1
            if c:
                self.counts[old] = c
            else:
                del self.counts[old]
        self.window.append(token)
        self.counts[token] = self.counts.get(token, 0) + 1

    def counts_before_unknown(self) -> Dict[int, int]:
        """The counts of the window as they will stand when one more token, not known yet, has
        entered it: without that token itself, but with the oldest token gone if the window
        is full."""
        n = self.params.repeat_last_n
        if n <= 0 or len(self.window) < n:
            return self.counts
        out = dict(self.counts)
        old = self.window[0]
        if out[old] > 1:
            out[old] -= 1
        else:
            del out[old]
        return out

    def next_uniform(self) -> float:
        return 0.0 if self.params.greedy else self.rng.next_f64()


STATUS_WORDS = 4     # the library's status words travel in front of the tokens


class PendingTokens:
    """Tokens that the device has drawn (or will, in stream order) and the host has not read."""

    def __init__(self, event, host: torch.Tensor, rows: int):
        self._event, self._host, self.rows = event, host, rows
        self.status: Optional[List[int]] = None

    def result(self) -> List[int]:
        """Wait for the draw and return the token ids.  Afterwards ``status`` holds the
        library's status words as they stood when the tokens were drawn (all zero when every
        kernel before the draw ran to its end)."""
        self._event.synchronize()
        words = self._host[:STATUS_WORDS + self.rows].tolist()
        self.status = words[:STATUS_WORDS]
        return words[STATUS_WORDS:]


class DeviceSampler:
    """Samples one token for each row of a logits tensor on the device."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._cap = 0
        self.h2d_bytes = 0       # bytes copied to and from the device so far
        self.d2h_bytes = 0

    def _buffers(self, rows: int, triples: int):
        need = max(rows, 1)
        if need > self._cap:
            self._cap = max(64, 2 * need)
            c = self._cap
            # host (pinned) and device copies of the per-row options, packed in one buffer:
            # [temperature f32 | top_p f32 | min_p f32 | repeat f32 | freq f32 | presence f32 |
            #  top_k i32 | pad | uniform f64]
            # (two host copies in turn, each with the event of its last copy to the device: a
            # draw may be prepared while the copy for the one before it is still queued)
            self._host = [torch.empty(c * 10, dtype=torch.float32, pin_memory=True)
                          for _ in range(2)]
            self._host_key = [None, None]
            self._host_event = [None, None]
            self._dev = torch.empty(c * 10, dtype=torch.float32, device=self.device)
            self._dev_key = None
            # [status words | tokens]: one copy brings both to the host
            self._out = torch.zeros(STATUS_WORDS + c, dtype=torch.int32, device=self.device)
            # two host copies in turn: a draw may be launched before the one before it is read
            self._out_host = [torch.empty(STATUS_WORDS + c, dtype=torch.int32, pin_memory=True)
                              for _ in range(2)]
            self._flip = 0
        if triples:
            if getattr(self, "_tri_cap", 0) < triples:
                self._tri_cap = max(1024, 2 * triples)
                self._tri_host = torch.empty(self._tri_cap * 3, dtype=torch.int32,
                                             pin_memory=True)
                self._tri_dev = torch.empty(self._tri_cap * 3, dtype=torch.int32,
                                            device=self.device)

    @property
    def device_tokens(self) -> torch.Tensor:
        """The int32 device buffer whose first rows hold the tokens of the latest draw."""
        return self._out[STATUS_WORDS:]

    def sample(self, logits: torch.Tensor, samplers: Sequence[RequestSampler]) -> List[int]:
        """``logits`` float32 [rows, vocab] on the device (modified in place by penalties);
        one :class:`RequestSampler` per row.  Returns the sampled token ids."""
        if logits.shape[0] == 0:
            return []
        return self.launch(logits, samplers).result()

    def launch(self, logits: torch.Tensor, samplers: Sequence[RequestSampler],
               inflight: Optional[Sequence[int]] = None) -> PendingTokens:
        """As :meth:`sample` without waiting: the draw and the copy of the tokens to the host
        are queued on the stream; at most two draws may be unread at a time.  ``inflight``: per
        row, the row of the draw before this one (:attr:`device_tokens`) whose token enters this
        row's penalty window although the host has not seen it yet, or -1: the step before is
        still running and this row's input is the token it draws."""
        rows = logits.shape[0]
        assert rows == len(samplers) and logits.dtype == torch.float32 and rows > 0
        tri: List[int] = []
        src: List[int] = [-1] * rows
        for r, s in enumerate(samplers):
            if s.params.penalties_active:
                unknown = inflight is not None and inflight[r] >= 0
                if unknown:
                    src[r] = int(inflight[r])
                for tok, cnt in (s.counts_before_unknown() if unknown else s.counts).items():
                    tri += (r, tok, cnt)
        any_unknown = any(x >= 0 for x in src)
        # (the tokens of the draw before, taken before the buffers may be replaced by larger ones)
        drawn = self.device_tokens if any_unknown else None
        self._buffers(rows, len(tri) // 3 + (rows if any_unknown else 0))
        c = self._cap
        # the options of a row change only when the set of requests changes; the uniforms
        # change with every draw (greedy rows draw nothing)
        key = [s.serial for s in samplers]
        any_draw = any(not s.params.greedy for s in samplers)
        if key != self._dev_key or any_draw:
            i = self._flip
            if self._host_event[i] is not None:
                self._host_event[i].synchronize()
            h = self._host[i].numpy()
            if key != self._host_key[i]:
                f = h[:6 * c].reshape(6, c)
                k = h[6 * c:7 * c].view(np.int32)
                for r, s in enumerate(samplers):
                    p = s.params
                    f[0, r], f[1, r], f[2, r] = p.temperature, p.top_p, p.min_p
                    f[3, r], f[4, r], f[5, r] = (p.repeat_penalty, p.frequency_penalty,
                                                 p.presence_penalty)
                    k[r] = p.top_k
                self._host_key[i] = key
            u = h[8 * c:10 * c].view(np.float64)
            for r, s in enumerate(samplers):
                u[r] = s.next_uniform()
            self._dev.copy_(self._host[i], non_blocking=True)
            self.h2d_bytes += self._host[i].numel() * 4
            self._host_event[i] = torch.cuda.Event()
            self._host_event[i].record()
            self._dev_key = key
        d = self._dev
        if tri or any_unknown:
            n = len(tri) // 3
            # the rows' sources of tokens in flight travel behind the triples
            words = tri + (src if any_unknown else [])
            if getattr(self, "_tri_event", None) is not None:
                self._tri_event.synchronize()       # the copy of the draw before has left
            self._tri_host[:len(words)] = torch.tensor(words, dtype=torch.int32)
            self._tri_dev[:len(words)].copy_(self._tri_host[:len(words)], non_blocking=True)
            self.h2d_bytes += 4 * len(words)
            self._tri_event = torch.cuda.Event()
            self._tri_event.record()
            kernels.apply_penalties(logits, self._tri_dev, n, d[3 * c:4 * c], d[4 * c:5 * c],
                                    d[5 * c:6 * c],
                                    self._tri_dev[3 * n:3 * n + rows] if any_unknown else None,
                                    drawn)
        kernels.sample(logits, d[0:c], d[6 * c:7 * c].view(torch.int32), d[c:2 * c],
                       d[2 * c:3 * c], d[8 * c:10 * c].view(torch.float64),
                       self._out[STATUS_WORDS:], self._out[:STATUS_WORDS])
        host = self._out_host[self._flip]
        self._flip ^= 1
        n = STATUS_WORDS + rows
        host[:n].copy_(self._out[:n], non_blocking=True)
        self.d2h_bytes += 4 * n
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(event, host, rows)
