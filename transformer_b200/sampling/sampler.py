"""Sampling on the device: one kernel launch for all rows of a step."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..csrc import lib
from .args import SampleArgs


class Sampler:
    def __init__(self, device: torch.device, max_rows: int = 1024):
        self.device = device
        self._idx = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._val = torch.empty(max_rows, dtype=torch.float32, device=device)
        self._u = torch.empty(max_rows, dtype=torch.float32, device=device)
        self._u_host = torch.empty(max_rows, dtype=torch.float32, pin_memory=True)
        self._event = torch.cuda.Event()

    def _grow(self, rows: int) -> None:
        if rows > self._idx.numel():
            torch.cuda.synchronize(self.device)
            self.__init__(self.device, max(rows, 2 * self._idx.numel()))

    def sample(self, logits: torch.Tensor, args: SampleArgs, u: Optional[Sequence[float]] = None):
        """logits: float [rows, vocab] on the device.  Returns (ids int32 [rows], values float [rows]),
        device tensors that the next call overwrites."""
        rows, V = logits.shape
        if logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise ValueError("the sampler reads float32 logits with contiguous rows")
        self._grow(rows)
        if not args.greedy:
            if u is None or len(u) != rows:
                raise ValueError("sampling with a temperature needs one uniform number per row")
            self._event.synchronize()
            self._u_host[:rows] = torch.tensor(list(u), dtype=torch.float32)
            self._u[:rows].copy_(self._u_host[:rows], non_blocking=True)
            self._event.record()
        lib.call("tb_sample", lib.ptr(logits), logits.stride(0), lib.ptr(self._u), rows, V,
                 float(args.temperature), int(args.top_k), float(args.top_p), lib.ptr(self._idx),
                 lib.ptr(self._val))
        return self._idx[:rows], self._val[:rows]
