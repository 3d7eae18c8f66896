"""Per-request sampling and stopping options, with the reference's names, meanings and defaults
(crates/engine/src/session.rs:14-41; DOCS.md "Request fields")."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    max_tokens: int = 64
    temperature: float = 1.0             # 0: greedy
    top_p: float = 0.95
    top_k: int = 20                      # 0: the whole candidate pool; 1: greedy
    min_p: float = 0.0                   # drops candidates below min_p times the most likely one's probability
    presence_penalty: float = 0.0        # subtracted from the logits of tokens already generated
    repetition_penalty: float = 1.0      # divides positive (multiplies negative) logits of generated tokens
    seed: Optional[int] = None           # None: drawn at random when the request is added
    stop_tokens: List[int] = field(default_factory=list)   # generation ends after any of these (which is emitted)

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if not 0 <= self.min_p <= 1:
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    @property
    def penalized(self) -> bool:
        return self.presence_penalty != 0.0 or self.repetition_penalty != 1.0

    @classmethod
    def greedy_params(cls, max_tokens: int = 64, stop_tokens=()) -> "SamplingParams":
        return cls(max_tokens=max_tokens, temperature=0.0, stop_tokens=list(stop_tokens))
