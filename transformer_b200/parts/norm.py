"""RMSNorm fused with the residual sum (models/llama/common/src/compute.rs:207,275,362)."""
from __future__ import annotations

from ..csrc import lib
from .base import NORMS, Norm, ParamDecl, WeightedRows


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: width, eps.  Statistics and the residual sum are float; one rounding at the store."""

    graph_safe = True
    launches_only = True
    takes_weighted_rows = True
    can_warm = True
    tails = ("router",)

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.width = int(params["width"])
        self.eps = float(params["eps"])

    def parameters(self):
        return {"weight": ParamDecl((self.width,), "norm", "ones")}

    def forward(self, ctx, x, delta, rows, y, warm=None, tail=None) -> None:
        n_out = y.shape[0]
        wy = idx = wts = None
        k = 0
        if isinstance(delta, WeightedRows):
            wy, idx, wts, k, delta = delta.rows, delta.index, delta.weights, delta.k, None
        if tail is not None:
            # the router of the normalized rows in the same kernel; what that form does not take (many rows, odd
            # widths) gets the norm alone and the router's own kernel
            E = tail.weights.shape[0]
            sfx = lib.suffix(self.dtype)
            if lib.try_call("tb_add_rmsnorm_router_" + sfx, lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
                            lib.ptr(wts), k, lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps, lib.ptr(y),
                            lib.ptr(tail.weights), lib.ptr(tail.index), lib.ptr(tail.scores), n_out, self.width, E,
                            tail.k):
                return
            lib.call("tb_add_rmsnorm_" + sfx, lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx), lib.ptr(wts), k,
                     lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps, lib.ptr(y), n_out, self.width,
                     lib.ptr(tail.weights), tail.weights.numel() * tail.weights.element_size())
            lib.call("tb_router_" + sfx, lib.ptr(y), lib.ptr(tail.weights), lib.ptr(tail.index), lib.ptr(tail.scores),
                     0, 0, 0, 0, 0, n_out, self.width, E, tail.k)
            return
        lib.call("tb_add_rmsnorm_" + lib.suffix(self.dtype), lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
                 lib.ptr(wts), k, lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps, lib.ptr(y), n_out,
                 self.width, lib.ptr(warm), 0 if warm is None else warm.numel() * warm.element_size())
