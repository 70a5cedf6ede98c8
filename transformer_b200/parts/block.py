"""The arrangement of a layer's parts in a block.

"pre_norm" (models/llama/common/src/compute.rs:204-336):

    x += mixer(norm_m(x));   x += feed_forward(norm_f(x))

The residual stream ``x`` is float.  A part writes its contribution ``delta``; the sum into ``x``
is fused into the NEXT norm (of this block or the following one, or the final norm), so a block
takes the pending delta of the block before it and returns its own.

Arrangements are registered like parts (:data:`ARRANGEMENTS`): a class built from (LayerSpec, dtype, device)
that offers ``parts()`` (name -> part: the names under which the weights are bound), ``mixer`` (whose cache
and state needs the engine serves) and ``forward(ctx, x, pending, cache_view, state)`` with the contract
above: ``pending`` is what the block before left to be added to ``x`` (a tensor, a WeightedRows, or None), the
return value is what this block leaves.  A block that wants its sums done at once can call
:func:`add_pending` and return None.
"""
from __future__ import annotations

from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, WeightedRows


def build_layer(spec, dtype, device):
    """The block of one LayerSpec, by its arrangement."""
    return ARRANGEMENTS.get(spec.arrangement)(spec, dtype, device)


@ARRANGEMENTS.register("pre_norm")
class Layer:
    """The parts of one LayerSpec, built, in the pre-norm arrangement."""

    def __init__(self, spec, dtype, device):
        if spec.mixer_norm is None or spec.feed_forward_norm is None:
            raise ValueError("the pre_norm arrangement needs a norm before the mixer and one before the feed-forward")
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts().values())

    @property
    def launches_only(self) -> bool:
        return all(p.launches_only for p in self.parts().values())

    def parts(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "feed_forward_norm": self.feed_forward_norm, "feed_forward": self.feed_forward}

    def forward(self, ctx, x, pending, cache_view, state):
        """x: float [nt, d]; pending: the previous block's delta or None.  Returns this block's
        pending delta (the feed-forward's output)."""
        nt, d = x.shape
        x1 = ctx.scratch("block.x1", (nt, d), ctx.dtype)
        delta = ctx.scratch("block.delta", (nt, d), ctx.dtype)
        pending = resolve(pending, self.mixer_norm, delta)
        self._norm(self.mixer_norm, self.mixer, ctx, x, pending, x1)
        self.mixer.forward(ctx, x1, delta, cache_view, state)
        tail = self.feed_forward.norm_tail(ctx, nt)
        if tail is not None and tail.kind in self.feed_forward_norm.tails:
            # the feed-forward's first small step rides along with the norm before it
            self.feed_forward_norm.forward(ctx, x, delta, None, x1, tail=tail)
            lazy = self.feed_forward.forward(ctx, x1, delta, tail=tail)
        else:
            self._norm(self.feed_forward_norm, self.feed_forward, ctx, x, delta, x1)
            lazy = self.feed_forward.forward(ctx, x1, delta)
        return delta if lazy is None else lazy


    @staticmethod
    def _norm(norm, then, ctx, x, delta, y) -> None:
        """The norm before the part ``then``; a norm that can do so starts fetching what that part reads first."""
        early = then.early_weights() if norm.can_warm else None
        if early is not None:
            norm.forward(ctx, x, delta, None, y, warm=early)
        else:
            norm.forward(ctx, x, delta, None, y)


def add_pending(ctx, x, pending) -> None:
    """x += pending, at once and in float, for an arrangement that does not leave the sum to a norm."""
    if pending is None:
        return
    if isinstance(pending, WeightedRows):
        from .feed_forward import sum_weighted_rows
        into = ctx.scratch("block.delta", tuple(x.shape), ctx.dtype)
        sum_weighted_rows(pending, into)
        pending = into
    x.add_(pending.float())


def resolve(pending, norm, into):
    """A pending WeightedRows stays as it is for a norm that sums it itself; else it is summed into ``into``."""
    if isinstance(pending, WeightedRows) and not norm.takes_weighted_rows:
        from .feed_forward import sum_weighted_rows
        sum_weighted_rows(pending, into)
        return into
    return pending
