"""Sampling options, with the reference's names, defaults and meanings
(crates/braidinfer-runtime/src/sampling.rs:7-47)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0          # 0.0 means argmax; otherwise logits are divided by it
    top_k: int = 50                   # keep the k largest logits; 0 disables
    top_p: float = 1.0                # nucleus: smallest set of largest probabilities reaching top_p
    repetition_penalty: float = 1.0   # > 1 lowers tokens already in the sequence, once per occurrence
    seed: Optional[int] = None        # None: a seed from the operating system
    min_p: float = 0.0                # drop tokens whose probability is below min_p * the largest
    logit_bias: Optional[Tuple[Tuple[int, float], ...]] = None   # (token, delta) added before all else

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be positive, got {self.repetition_penalty}")
        if self.logit_bias is not None:
            object.__setattr__(self, "logit_bias", tuple((int(t), float(d)) for t, d in self.logit_bias))

    @classmethod
    def greedy(cls) -> "SamplingParams":
        """The reference's `SamplingParams::greedy()` (sampling.rs:35-46)."""
        return cls(temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=None, min_p=0.0,
                   logit_bias=None)

    @property
    def is_plain_greedy(self) -> bool:
        return self.temperature == 0.0 and self.repetition_penalty == 1.0 and not self.logit_bias
