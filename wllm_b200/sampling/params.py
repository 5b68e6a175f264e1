"""Sampling options of a request.

The first six fields and their defaults are the reference's (src/wllm/engine/sampling.py:22-29):
temperature 0 means greedy; top_k 0, top_p 1, min_p 0 and repetition_penalty 1 switch
their filter off.  The reference accepts `seed` and ignores it; here a seeded request
draws the same tokens whatever else is in the batch and however its prompt was cut,
because the draw for output place i depends on (seed, i) only.  The rest are the
request-level fields the reference keeps on its Sequence
(src/wllm/engine/sequence.py:25-27): max_tokens (max_new_tokens), stop_token_ids, and
ignore_eos (ours).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    seed: int | None = None
    max_tokens: int = 16
    stop_token_ids: tuple = ()
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0 (0 = greedy)")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0 = off)")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1] (1 = off)")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1] (0 = off)")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0 (1 = off)")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        object.__setattr__(self, "stop_token_ids", tuple(self.stop_token_ids))

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


_MASK = (1 << 64) - 1


def uniform_from(seed: int, counter: int) -> float:
    """The kernel's uniform draw for (seed, output place), restated for the host and the tests."""
    z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0
