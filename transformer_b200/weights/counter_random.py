"""Random numbers that are a pure function of (seed, tensor name, element index).

Random weights drawn from a generator's stream depend on who draws them and in which order: a CPU
generator, a CUDA generator and a test's own code never agree.  Here element ``i`` of the tensor
``name`` is computed from a counter, so a file writer on the CPU, a fill kernel on the GPU
(``csrc/random_fill.cu``) and any restatement give the same bits:

    base  = mix64((seed * G + fnv1a64(name)) mod 2^64)          G = 0x9E3779B97F4A7C15
    h0, h1 = mix64(base + (2i) * G), mix64(base + (2i + 1) * G)  (mod 2^64; mix64 = splitmix64's finalizer)
    c     = sum of the eight 16-bit fields of h0 and h1, minus 4 * 65535
    value = float32(c) * float32(std / SIGMA)                    SIGMA = sqrt(8 * (2^32 - 1) / 12)

The sum of eight uniform integers is close to a normal variable (it ends at 4.9 standard deviations);
``c`` is an integer below 2^24, so its conversion is exact and the product is the only rounding.  The
value is rounded to the storage type afterwards.  The reference draws no weights: it reads files only
(models/llama/common/src/storage.rs:29-88).
"""
from __future__ import annotations

import math

import numpy as np

G = 0x9E3779B97F4A7C15
MASK = (1 << 64) - 1
SIGMA = math.sqrt(8.0 * ((1 << 32) - 1) / 12.0)


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & MASK
    return h


def mix64_int(z: int) -> int:
    z &= MASK
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & MASK
    z ^= z >> 31
    return z


def stream_base(seed: int, name: str) -> int:
    """Where the stream of tensor ``name`` starts for this seed."""
    return mix64_int((int(seed) * G + fnv1a64(name)) & MASK)


def scale_for(std: float) -> np.float32:
    return np.float32(std / SIGMA)


def _mix64(z: np.ndarray) -> np.ndarray:
    z = z ^ (z >> np.uint64(30))
    z = z * np.uint64(0xBF58476D1CE4E5B9)
    z = z ^ (z >> np.uint64(27))
    z = z * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def normal_values(seed: int, name: str, first: int, count: int, std: float) -> np.ndarray:
    """float32 values of elements first .. first + count - 1 of tensor ``name``."""
    out = np.empty(count, dtype=np.float32)
    base, scale = np.uint64(stream_base(seed, name)), scale_for(std)
    with np.errstate(over="ignore"):
        for lo in range(0, count, 1 << 22):            # in slabs: a handful of temporaries of 32 MB each
            n = min(1 << 22, count - lo)
            i2 = (np.arange(first + lo, first + lo + n, dtype=np.uint64) * np.uint64(2))
            total = np.zeros(n, dtype=np.int64)
            for j in (0, 1):
                h = _mix64(base + (i2 + np.uint64(j)) * np.uint64(G))
                for f in range(4):
                    total += ((h >> np.uint64(16 * f)) & np.uint64(0xFFFF)).astype(np.int64)
            out[lo:lo + n] = (total - 4 * 65535).astype(np.float32) * scale
    return out
