"""Feed-forward parts: a dense SwiGLU and a softmax-top-k mixture of SwiGLU experts.

The reference runs the experts as a host loop over tokens and chosen experts with one product
each and a device-to-host copy of the router logits in every layer
(models/llama/common/src/compute.rs:294-333).  Here the tokens are sorted by expert on the device
and every expert runs once over all of its tokens (a grouped product); nothing touches the host.
"""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import FEED_FORWARDS, FeedForward, NormTail, ParamDecl, WeightedRows
from . import linear
from .linear import gemm_skinny, grouped_matmul, matmul_nt

ROUTER_ROWS_FROM = 256      # above this many tokens the router works on tiles of 16 tokens (tensor cores)
ROUTER_TAIL_ROWS = 256      # up to this many tokens the norm before the experts also routes


@FEED_FORWARDS.register("swiglu")
class DenseSwiGLU(FeedForward):
    """params: width, di.  gate_up = x1 Wgu^T (gate rows first), h = silu(gate) * up, out = h Wd^T
    (compute.rs:278-292)."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])
        self.di = int(params["di"])

    def parameters(self):
        return {"wgu": ParamDecl((2 * self.di, self.d)), "wd": ParamDecl((self.d, self.di))}

    def forward(self, ctx, x1, out) -> None:
        nt = x1.shape[0]
        h = ctx.scratch("ff.h", (nt, self.di), self.dtype)
        grouped_matmul(x1, self.weights["wgu"], h, swiglu=True)
        matmul_nt(h, self.weights["wd"], out)


@FEED_FORWARDS.register("moe")
class MoE(FeedForward):
    """params: width, di, nexp, nexp_use.

    router logits (float) -> the nexp_use largest, equal logits to the lower expert -> softmax over
    the kept logits (compute.rs:375-394) -> expert SwiGLU (compute.rs:320-328) -> weighted sum in
    descending-logit order, in float (compute.rs:329-330)."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])
        self.di = int(params["di"])
        self.E = int(params["nexp"])
        self.k = int(params["nexp_use"])
        if not (0 < self.k <= self.E):
            raise ValueError(f"experts per token {self.k} must lie in 1..{self.E}")
        if self.E > 1024:
            raise ValueError(f"the routing kernels take up to 1024 experts, got {self.E}")

    def parameters(self):
        return {
            "router": ParamDecl((self.E, self.d)),
            "wgu": ParamDecl((self.E, 2 * self.di, self.d)),
            "wd": ParamDecl((self.E, self.d, self.di)),
        }

    def early_weights(self):
        """The router's matrix: small, and every token's block waits for all of it."""
        r = self.weights.get("router")
        return r if r is not None and r.numel() * r.element_size() <= (1 << 20) else None

    def route(self, ctx, x1, logits_out=None, lists=None):
        """Experts and weights of every token.  With ``lists`` = (offsets, sorted_token, pair_row) the dispatch lists
        are wanted too; returns (idx, w, whether the lists were built along the way)."""
        nt = x1.shape[0]
        idx = ctx.scratch("moe.topk_idx", (nt, self.k), torch.int32)
        w = ctx.scratch("moe.topk_w", (nt, self.k), torch.float32)
        if self.dtype == torch.bfloat16 and nt > ROUTER_ROWS_FROM and self.E <= 64:
            # many tokens, few experts: 16 tokens' logits are a tensor-core tile, the activations are read once, and
            # the block that finishes last builds the dispatch lists
            done = ctx.scratch("moe.done", (1,), torch.int32, zero=True) if lists is not None else None
            offsets, sorted_token, pair_row = lists if lists is not None else (None, None, None)
            if lib.try_call("tb_router_rows_bf16", lib.ptr(x1), lib.ptr(self.weights["router"]), lib.ptr(idx), lib.ptr(w),
                            lib.ptr(logits_out), lib.ptr(offsets), lib.ptr(sorted_token), lib.ptr(pair_row),
                            lib.ptr(done), nt, self.d, self.E, self.k):
                return idx, w, lists is not None
        # a few tokens: the block that finishes last builds the lists, which saves a kernel on the way to the experts
        fused = lists is not None and nt <= ROUTER_ROWS_FROM
        done = ctx.scratch("moe.done", (1,), torch.int32, zero=True) if fused else None
        offsets, sorted_token, pair_row = lists if fused else (None, None, None)
        lib.call("tb_router_" + lib.suffix(self.dtype), lib.ptr(x1), lib.ptr(self.weights["router"]),
                 lib.ptr(idx), lib.ptr(w), lib.ptr(logits_out), lib.ptr(offsets), lib.ptr(sorted_token),
                 lib.ptr(pair_row), lib.ptr(done), nt, self.d, self.E, self.k)
        return idx, w, fused

    def norm_tail(self, ctx, nt):
        """For a few tokens the router rides along with the norm before this part."""
        if nt > ROUTER_TAIL_ROWS:
            return None
        return NormTail("router", weights=self.weights["router"], k=self.k,
                        index=ctx.scratch("moe.topk_idx", (nt, self.k), torch.int32),
                        scores=ctx.scratch("moe.topk_w", (nt, self.k), torch.float32))

    def forward(self, ctx, x1, out, tail=None) -> None:
        nt = x1.shape[0]
        M = nt * self.k
        sfx = lib.suffix(self.dtype)
        if self.dtype == torch.bfloat16 and M <= linear.SKINNY_MAX_PAIRS and self.d % 8 == 0 and self.di % 8 == 0:
            # a few tokens: no dispatch lists.  Row p = t * k + j of the experts' products is the pair (token t,
            # its j-th choice); every block of the product kernel finds its expert's pairs in the router's answer
            idx, w = (tail.index, tail.scores) if tail is not None else self.route(ctx, x1)[:2]
            h = ctx.scratch("moe.h", (M, self.di), self.dtype)
            y = ctx.scratch("moe.y", (M, self.d), self.dtype)
            pairs = idx.view(-1)
            if gemm_skinny(x1, self.weights["wgu"], h, groups=self.E, out_kind=2, max_group_rows=nt, row_group=pairs,
                           x_div=self.k) and \
                    gemm_skinny(h, self.weights["wd"], y, groups=self.E, max_group_rows=nt, row_group=pairs):
                ctx.record("moe.topk_idx", idx)
                return WeightedRows(y, _identity_rows(M, x1.device), w, self.k)
        offsets = ctx.scratch("moe.offsets", (self.E + 1,), torch.int32)
        sorted_token = ctx.scratch("moe.sorted_token", (M,), torch.int32)
        pair_row = ctx.scratch("moe.pair_row", (M,), torch.int32)
        if tail is not None:
            idx, w, listed = tail.index, tail.scores, False
        else:
            idx, w, listed = self.route(ctx, x1, lists=(offsets, sorted_token, pair_row))
        ctx.record("moe.topk_idx", idx)
        if not listed:
            lib.call("tb_moe_dispatch", lib.ptr(idx), lib.ptr(offsets), lib.ptr(sorted_token), lib.ptr(pair_row),
                     M, self.k, self.E)
        h = ctx.scratch("moe.h", (M, self.di), self.dtype)
        grouped_matmul(x1, self.weights["wgu"], h, a_rows=sorted_token, group_offsets=offsets, groups=self.E,
                       swiglu=True, max_group_rows=nt, scratch=ctx.scratch)
        y = ctx.scratch("moe.y", (M, self.d), self.dtype)
        grouped_matmul(h, self.weights["wd"], y, group_offsets=offsets, groups=self.E, max_group_rows=nt)
        # the weighted sum over the chosen experts is left to the norm that follows (fused there)
        return WeightedRows(y, pair_row, w, self.k)


_IDENTITY_ROWS = {}


def _identity_rows(n: int, device) -> torch.Tensor:
    """0 .. n-1 as int32, made once per size."""
    key = (n, str(device))
    if key not in _IDENTITY_ROWS:
        _IDENTITY_ROWS[key] = torch.arange(n, dtype=torch.int32, device=device)
    return _IDENTITY_ROWS[key]


def sum_weighted_rows(wr: WeightedRows, out) -> None:
    """out[t] = sum_j weights[t, j] * rows[index[t, j]], for a consumer that wants a plain tensor."""
    nt, d = out.shape
    lib.call("tb_moe_combine_" + lib.suffix(out.dtype), lib.ptr(wr.rows), lib.ptr(wr.index), lib.ptr(wr.weights),
             lib.ptr(out), nt, d, wr.k)
