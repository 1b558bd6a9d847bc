"""Sampling options, with the reference's names, meanings and defaults
(src/main.c:65-94, 273 of AnonymoDGH/gguf2bin): ``-t`` temperature 0.7 (0 = greedy),
``--top-k`` 40, ``--top-p`` 0.9, ``--repeat-penalty`` 1.1 over the last 64 tokens."""
from __future__ import annotations

from dataclasses import dataclass

RECENT_USE = 64          # tokens the repeat penalty looks back over (src/main.c:18)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    repeat_penalty: float = 1.1

    def __post_init__(self):
        if not (self.top_p > 0.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if not (self.repeat_penalty > 0.0):
            raise ValueError(f"repeat_penalty must be positive, got {self.repeat_penalty}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def filtered(self) -> bool:
        """True when top-k, top-p or the repeat penalty changes anything; otherwise the
        plain sampler (src/l5_model.c:608-620) is the whole of it."""
        return self.repeat_penalty != 1.0 or (not self.greedy and
                                              (self.top_k > 0 or self.top_p < 1.0))

    @staticmethod
    def plain(temperature: float = 0.0) -> "SamplingParams":
        """Greedy or temperature sampling alone."""
        return SamplingParams(temperature=temperature, top_k=0, top_p=1.0, repeat_penalty=1.0)
