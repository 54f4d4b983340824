"""Sampling options, with the reference's names, meanings and defaults
(``GenerationConfig``, crates/synaptix-models/llm/common/src/generate.rs:16-57)."""
from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0        # <= 0: greedy argmax; else logits /= temperature, then a draw
    top_k: int = 0                  # 0 = off; keep the k largest
    top_p: float = 1.0              # >= 1 = off; smallest prefix of the sorted probabilities whose sum passes p
    min_p: float = 0.0              # 0 = off; drop probabilities below min_p * the largest
    repetition_penalty: float = 1.0  # 1 = off; per occurrence in the window: logit > 0 ? /p : *p
    repeat_last_n: int = 0          # window of the penalties in tokens of context; 0 = all of it
    presence_penalty: float = 0.0   # subtracted once per distinct token of the window
    frequency_penalty: float = 0.0  # subtracted times the token's count in the window
    seed: int = 0                   # key of the Philox stream

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0)

    @property
    def penalties_on(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.presence_penalty != 0.0
                or self.frequency_penalty != 0.0)

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (self.top_p > 0.0):
            raise ValueError("top_p must be > 0")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must lie in [0, 1]")
        if not (self.repetition_penalty > 0.0):
            raise ValueError("repetition_penalty must be > 0")
        if self.repeat_last_n < 0:
            raise ValueError("repeat_last_n must be >= 0")
