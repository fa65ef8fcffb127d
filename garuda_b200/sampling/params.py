"""How logits become a token: the options of the reference, with its defaults.

garuda/src/runtime/mod.rs:15-39: ``temperature`` 0 is greedy (the other knobs are
then ignored), else logits are divided by it; ``top_k`` keeps the k most likely
(0: off); ``top_p`` keeps the shortest prefix of the sorted list whose
probability reaches it (1: off); ``max_tokens`` caps the generation; ``seed``
pins the generator, and without one the request's id does (:612).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

from ..config.model_config import ConfigError


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8
    top_p: float = 0.95
    top_k: int = 40
    max_tokens: int = 128
    seed: Optional[int] = None

    def validate(self) -> None:
        """garuda/src/runtime/mod.rs:42-59."""
        if not math.isfinite(self.temperature) or self.temperature < 0:
            raise ConfigError(f"temperature must be a non-negative number, got {self.temperature}")
        if not math.isfinite(self.top_p) or self.top_p <= 0 or self.top_p > 1:
            raise ConfigError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ConfigError(f"top_k must not be negative, got {self.top_k}")
        if self.max_tokens < 1:
            raise ConfigError("max_tokens must be at least 1")

    @classmethod
    def greedy(cls, max_tokens: int = 128) -> "SamplingParams":
        return cls(temperature=0.0, top_p=1.0, top_k=0, max_tokens=max_tokens)
