"""Per-request sampling options: the reference's names, meanings and defaults
(crates/engine/decode/src/params.rs:12-67)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0        # <= 0: greedy (arg max of the processed logits)
    top_k: int = 40                 # keep the k highest logits; <= 0 disables
    top_p: float = 0.95             # smallest prefix with cumulative probability >= top_p; >= 1 disables
    min_p: float = 0.05             # drop p < min_p * p_max; <= 0 disables
    repeat_penalty: float = 1.0     # over the last repeat_last_n tokens, prompt included; 1 disables
    repeat_last_n: int = 64         # 0 disables the three penalties
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None      # None: drawn from the operating system
    max_tokens: int = 4096          # generation cap (crates/engine/server/src/api.rs:340-344)
    ignore_eos: bool = False        # keep generating past an end-of-sequence token (benchmarks)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def penalties_active(self) -> bool:
        return self.repeat_last_n > 0 and (self.repeat_penalty != 1.0 or
                                           self.frequency_penalty != 0.0 or
                                           self.presence_penalty != 0.0)

    @classmethod
    def greedy_params(cls, max_tokens: int = 4096, **kw) -> "SamplingParams":
        return cls(temperature=0.0, max_tokens=max_tokens, **kw)
