"""How the next token is chosen. Names, defaults and checks follow the reference's `SamplingOptions`
(src/etalii_dllm/sampling.py:24-111): temperature 0 is greedy (the first index of the largest logit); above zero the
choice is drawn with a seeded generator, never from ambient entropy, so the same options, model and prompt give the
same tokens."""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class SamplingOptions:
    temperature: float = 0.0
    """0 means greedy decoding."""
    top_k: int = 0
    """Keep only the K most likely tokens; 0 disables."""
    top_p: float = 1.0
    """Nucleus threshold in (0, 1]; 1 disables."""
    seed: int = 0
    """Seed of the sampler's random stream (taken modulo 2^64). Sequence i of a request list draws from the stream
    of seed + i (the reference's rule for the choices of one prompt, sampling.py:161-164)."""
    min_p: float = 0.0
    """Drop candidates less likely than min_p times the most likely one; 0 disables."""

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be non-negative")
        if not 0 <= self.min_p <= 1:
            raise ValueError("min_p must be in [0, 1]")

    def for_choice(self, index: int) -> "SamplingOptions":
        return replace(self, seed=self.seed + index)
