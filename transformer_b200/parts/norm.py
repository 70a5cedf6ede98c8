"""RMSNorm fused with the residual sum (models/llama/common/src/compute.rs:207,275,362)."""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import NORMS, Norm, ParamDecl, WeightedRows


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: width, eps.  Statistics and the residual sum are float; one rounding at the store."""

    takes_weighted_rows = True
    can_warm = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.width = int(params["width"])
        self.eps = float(params["eps"])

    def parameters(self):
        return {"weight": ParamDecl((self.width,), "norm", "ones")}

    def forward(self, ctx, x, delta, rows, y, warm=None) -> None:
        n_out = y.shape[0]
        wy = idx = wts = None
        k = 0
        if isinstance(delta, WeightedRows):
            wy, idx, wts, k, delta = delta.rows, delta.index, delta.weights, delta.k, None
        lib.call("tb_add_rmsnorm_" + lib.suffix(self.dtype), lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
                 lib.ptr(wts), k, lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps, lib.ptr(y), n_out,
                 self.width, lib.ptr(warm), 0 if warm is None else warm.numel() * warm.element_size())
