"""The sampler's options, with the reference's names, meanings and defaults
(`SamplerParams`, alpacca/sample.py:12-19)."""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass
class SamplerParams:
    temperature: float = 0.8     # <= 0: greedy
    top_k: int = 40              # <= 0: the whole vocabulary
    top_p: float = 0.95          # outside (0, 1): no cut
    repeat_penalty: float = 1.1  # 1.0 or 0: off
    repeat_last_n: int = 64
    seed: int = -1               # -1 -> random

    def resolved_seed(self) -> int:
        if self.seed is not None and self.seed >= 0:
            return int(self.seed)
        return int.from_bytes(os.urandom(8), "little") >> 1

    @property
    def penalizes(self) -> bool:
        return bool(self.repeat_penalty) and self.repeat_penalty != 1.0

    @classmethod
    def greedy(cls) -> "SamplerParams":
        return cls(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=0)
