"""What a model needs from a weight file, as data.

A :class:`TensorRule` says: parameter ``dest`` has ``shape`` and ``role``, and is filled from one of
several alternative :class:`Source` s.  A source is a list of file tensors (by exact name, with the
shape each must have) and the way they are joined.  The first source is the canonical one: it is
what the random-weights writer produces and what an error message asks for.

Roles decide the storage type on the device:

* ``"matrix"``  -- follows the compute path: bfloat16 when serving, float32 on the 32-bit path
* ``"norm"``    -- always float32 (the reference keeps norm weights in f32,
                   docs/user-guide/doc.md:133 ``norm:f32``); a 32-bit tensor stays 32-bit
* ``"table"``   -- integers, kept as int32
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

Dest = Tuple  # e.g. ("layers", 3, "mixer", "wqkv")


@dataclass(frozen=True)
class Source:
    names: Tuple[str, ...]
    shapes: Tuple[Tuple[int, ...], ...]
    # "single" | "cat0" (concatenate along rows) | "cat1" (along dim 1) | "stack0" (a new leading dimension) |
    # "stack0_of_row_pairs" (parts a0, b0, a1, b1, ...: stack of cat0(a_i, b_i): per-expert gate and up matrices)
    join: str = "single"

    def combine(self, parts: Sequence[torch.Tensor]) -> torch.Tensor:
        if self.join == "single":
            return parts[0]
        if self.join == "cat0":
            return torch.cat(list(parts), dim=0)
        if self.join == "cat1":
            return torch.cat(list(parts), dim=1)
        if self.join == "stack0":
            return torch.stack(list(parts), dim=0)
        if self.join == "stack0_of_row_pairs":
            return torch.stack([torch.cat([parts[i], parts[i + 1]], dim=0) for i in range(0, len(parts), 2)], dim=0)
        raise ValueError(self.join)


@dataclass(frozen=True)
class TensorRule:
    dest: Dest
    shape: Tuple[int, ...]
    role: str                               # "matrix" | "norm" | "table"
    sources: Tuple[Source, ...]
    init: str = "normal"                    # how the random-weights mode fills it: "normal" | "ones"
    shared_with: Optional[Dest] = None      # when no source is present, reuse this parameter (tied head)

    @property
    def canonical(self) -> Source:
        return self.sources[0]


def single(name: str, shape: Sequence[int]) -> Source:
    return Source((name,), (tuple(shape),), "single")
