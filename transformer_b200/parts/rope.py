"""Rotary position encoding: the angle table (the rotation itself is fused with the cache write).

angle(p, i) = p * theta^(-2i/dh), i in [0, dh/2).  The reference builds sin/cos tables [nctx, dh]
once per model (models/llama/common/src/compute.rs:41-53, models/llama/cuda/src/infer.rs:89-90) and
passes theta along; pairing and the frequency formula are inside its external operator.  Here the
table is computed in double precision on the host and stored as float [positions, dh/2], so the
angle itself carries no 32-bit rounding at large positions.
"""
from __future__ import annotations

import torch

from .base import POSITIONS, Position

_TABLES = {}


@POSITIONS.register("rope")
class Rope(Position):
    """params: dh, theta, pairing ("adjacent" | "half"), positions (table length)."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.dh = int(params["dh"])
        self.theta = float(params["theta"])
        self.pairing = params.get("pairing", "adjacent")
        self.positions = int(params["positions"])
        if self.dh % 2:
            raise ValueError(f"rotary pairs need an even head size, got {self.dh}")
        if self.pairing not in ("adjacent", "half"):
            raise ValueError(f"unknown rope pairing {self.pairing!r}")

    @property
    def half_pairing(self) -> int:
        return 1 if self.pairing == "half" else 0

    def rotation(self):
        cos, sin = self.tables()
        return cos, sin, self.half_pairing

    def tables(self):
        key = (self.dh, self.theta, self.positions, str(self.device))
        if key not in _TABLES:
            i = torch.arange(self.dh // 2, dtype=torch.float64)
            inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.dh)
            ang = torch.arange(self.positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
            _TABLES[key] = (torch.cos(ang).float().contiguous().to(self.device),
                            torch.sin(ang).float().contiguous().to(self.device))
        return _TABLES[key]
