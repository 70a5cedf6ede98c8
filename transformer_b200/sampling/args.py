"""Sampling arguments and the per-sequence random numbers.

Names and meanings follow the reference's driver: TEMPERATURE (default 0 = argmax), TOP_P
(default 1), TOP_K (default unbounded), checked by ``SampleArgs::new`` before the model is built
(test-utils/src/lib.rs:78-80, models/llama/cuda/src/infer.rs:44).  The reference draws its uniform
number from the thread's generator (tensor/src/operators/random_sample.rs:72), so a run cannot be
repeated; here the number for the j-th token of request r under seed s is a pure function of
(s, r, j), whatever else is in the batch.
"""
from __future__ import annotations

from dataclasses import dataclass

_MASK = (1 << 64) - 1


class SampleArgsError(ValueError):
    pass


@dataclass(frozen=True)
class SampleArgs:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0          # 0 = no limit (the reference's default is usize::MAX)

    def __post_init__(self):
        if not (self.temperature >= 0.0) or self.temperature == float("inf"):
            raise SampleArgsError(f"temperature must lie in [0, inf), got {self.temperature}")
        if not (0.0 < self.top_p <= 1.0):
            raise SampleArgsError(f"top_p must lie in (0, 1], got {self.top_p}")
        if isinstance(self.top_k, bool) or int(self.top_k) != self.top_k or self.top_k < 0:
            raise SampleArgsError(f"top_k must be a non-negative integer (0 = no limit), got {self.top_k}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, request: int, index: int) -> float:
    """A number in [0, 1) with 24 random bits, fixed by (seed, request, index)."""
    h = _splitmix64(seed & _MASK)
    h = _splitmix64(h ^ ((request * 0xD1342543DE82EF95) & _MASK))
    h = _splitmix64(h ^ ((index * 0xA24BAED4963EE407) & _MASK))
    return (h >> 40) / float(1 << 24)
