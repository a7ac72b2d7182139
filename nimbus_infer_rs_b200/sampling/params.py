"""Sampling options, with the reference's names, meanings and defaults
(src/sampler.rs:7-35)."""
from __future__ import annotations

from dataclasses import dataclass, field

DEFAULT_SEED = 0x5DEECE66D  # used when no seed is given (src/engine.rs:271)


@dataclass
class SamplingParams:
    max_new_tokens: int = 64          # clipped to the context budget (src/engine.rs:265-266)
    temperature: float = 1.0          # <= 0 means greedy (src/sampler.rs:32-34)
    top_k: int = 0                    # 0 disables (src/sampler.rs:103-116)
    top_p: float = 1.0                # 1.0 disables (src/sampler.rs:118-160)
    repetition_penalty: float = 1.0   # 1.0 disables (src/sampler.rs:83-101)
    seed: int | None = None
    stop_tokens: list[int] = field(default_factory=list)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    def validate(self) -> None:
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if not self.repetition_penalty > 0:
            raise ValueError("repetition_penalty must be positive")
