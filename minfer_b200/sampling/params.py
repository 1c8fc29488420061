"""Sampling options, with the reference's names, meanings and defaults
(src/main.rs:42-70: temp 0.8, top-k 40, top-p 0.95, repeat penalty 1.1, frequency and
presence penalties 0, seed 42; temp 0 or --greedy means greedy)."""
from __future__ import annotations

from dataclasses import dataclass

RECENT_WINDOW = 64      # tokens the penalties look back over (src/main.rs:538)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    repeat_penalty: float = 1.1
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    seed: int = 42

    @classmethod
    def greedy(cls) -> "SamplingParams":
        """Pure greedy decoding: no penalties, the first maximum wins."""
        return cls(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0)

    @classmethod
    def pure_temperature(cls, temperature: float, seed: int = 42) -> "SamplingParams":
        return cls(temperature=temperature, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=seed)

    def validate(self) -> None:
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0 = off)")
        if not self.top_p > 0.0:
            raise ValueError("top_p must be > 0 (>= 1 = off)")
        if self.repeat_penalty <= 0.0:
            raise ValueError("repeat_penalty must be > 0 (1 = off)")
