"""The two ends of the model: token ids into the residual stream, normed rows into logits.

The reference's caller gathers embedding rows (models/llama/cuda/src/infer.rs:98-104,
test-utils/src/llama.rs:18-23) and its step ends with ``logits = x . output`` on the wanted rows
(models/llama/common/src/compute.rs:364-365; ``output`` is ``token_embd`` when the file has no
``output.weight``, storage.rs:84).  Here both are parts like any other: a model with a scaled
embedding, learned positions or capped logits registers another kind and the engine stays as it is.
"""
from __future__ import annotations

from ..csrc import lib
from .base import EMBEDDINGS, HEADS, Embedding, Head, ParamDecl
from .linear import matmul_nt


@EMBEDDINGS.register("lookup")
class Lookup(Embedding):
    """params: vocab, width.  x[i] = table[tok_i] as float, no scaling."""
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.vocab, self.width = int(params["vocab"]), int(params["width"])

    def parameters(self):
        return {"table": ParamDecl((self.vocab, self.width))}

    def forward(self, ctx, x) -> None:
        lib.call("tb_embed_" + lib.suffix(self.dtype), lib.ptr(ctx.tok_ids), lib.ptr(self.weights["table"]),
                 lib.ptr(x), x.shape[0], self.width)


@HEADS.register("linear")
class LinearHead(Head):
    """params: vocab, width, tied.  logits = xn weight^T in float, no bias, no scale, no cap.  ``tied``: the weight
    is the embedding's table unless the file holds one of its own (the weight plan's business, not this part's)."""
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.vocab, self.width = int(params["vocab"]), int(params["width"])

    def parameters(self):
        return {"weight": ParamDecl((self.vocab, self.width))}

    def forward(self, ctx, xn, logits) -> None:
        matmul_nt(xn, self.weights["weight"], logits)
