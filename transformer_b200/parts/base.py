"""Interfaces of the parts a layer is put together from, and one registry per kind of part.

A part is built from the parameters of its :class:`~transformer_b200.parts.spec.PartSpec` alone; it
does not know which model it is in, which layer it is, or what the other parts are.  The engine
talks to parts only through the methods below.

============  ===================================================================================
kind          interface
============  ===================================================================================
Embedding     ``forward(ctx, x)``: fill the float residual stream ``x`` [nt, d] for the step's tokens
              (``ctx.tok_ids``, and ``ctx.tok_pos`` for an encoding that adds positions here).
Norm          ``forward(ctx, x, delta, rows, y)``: ``v = x[rows] + delta[rows]`` (float sum; written
              back to ``x`` when ``rows`` is None), ``y = norm(v)``.  ``x`` is the float residual
              stream, ``delta`` the previous part's output or None.
Mixer         ``forward(ctx, x1, out, cache, state)``: reads the normed activations ``x1`` [nt, d]
              and writes its contribution to the stream into ``out`` [nt, d].  ``cache`` is what the
              storage class of its ``cache_need().kind`` shows a run (None if ``cache_need()`` is
              None), ``state`` its per-sequence state tensor [slots, *shape] (None if
              ``state_need()`` is None); rows of ``state`` are addressed by ``ctx.slots``.
FeedForward   ``forward(ctx, x1, out)``; may return a ``WeightedRows`` instead of filling ``out``.
Position      owned by the mixer that uses it.  A rotary encoding answers ``rotation()`` with its
              (cos, sin, half_pairing) and the mixer fuses the rotation with its cache write; any
              other encoding answers None and is called as ``apply(ctx, qkv, nh, nkvh, dh)`` to
              change the step's queries and keys in place by its own means.
Head          ``forward(ctx, xn, logits)``: float logits [rows, vocab] of the normed rows ``xn``.
Arrangement   how a layer's parts are put together in a block: built from a LayerSpec,
              ``parts()`` (name -> part), ``mixer``, ``forward(ctx, x, pending, cache, state)``.
============  ===================================================================================

All parts declare their parameters with :meth:`Part.parameters` (name -> shape, role, init) and
receive the device tensors with :meth:`Part.bind`.  A part whose ``forward`` only launches work on the
device that reads the step's numbers from ``ctx``'s DEVICE arrays (never from the ``h_*`` host lists,
never a value copied back to the host) may set ``graph_safe = True``: decode steps of a model whose
parts all say so are captured into CUDA graphs and replayed with new index arrays.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamDecl:
    shape: Tuple[int, ...]
    role: str = "matrix"     # "matrix" | "norm" | "table"
    init: str = "normal"     # "normal" | "ones"


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer wants kept for every sequence: ``kind`` names a registered storage class
    (:data:`transformer_b200.cache.paged.CACHE_KINDS`; "full" = keys and values of every position in pages),
    for nkvh heads of size dh; ``params`` holds what else the kind needs (a window's length, ...).  Runs with
    equal needs share one storage object."""
    kind: str
    nkvh: int
    dh: int
    params: Tuple[Tuple[str, Any], ...] = ()

    def get(self) -> Dict[str, Any]:
        return dict(self.params)


@dataclass(frozen=True)
class StateNeed:
    """A tensor of fixed size per sequence, zero when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class WeightedRows:
    """A part's output that is not summed yet: out[t] = sum_j weights[t, j] * rows[index[t * k + j]].
    A norm that sets ``takes_weighted_rows`` does the sum itself, in float, while it adds to the stream
    (one kernel and one round trip through memory less); for any other norm the block sums first."""
    rows: torch.Tensor        # [M, d]
    index: torch.Tensor       # int32 [nt * k]
    weights: torch.Tensor     # float [nt, k]
    k: int


class Part:
    graph_safe = False      # see the head of this file; the parts of this package set it
    launches_only = False   # all device work goes through csrc.lib launchers (or reports itself with lib.foreign):
                            # the engine may then record one layer's launches and replay them for its equals

    def __init__(self, params: Dict[str, Any], dtype: torch.dtype, device: torch.device):
        self.params = dict(params)
        self.dtype = dtype
        self.device = device
        self.weights: Dict[str, torch.Tensor] = {}

    def parameters(self) -> Dict[str, ParamDecl]:
        return {}

    def early_weights(self) -> Optional[torch.Tensor]:
        """A small weight that this part reads first and waits for (a router's matrix), or None.  The part that
        runs before it may ask for it to be brought into L2 meanwhile (``Norm.forward(..., warm=)``)."""
        return None

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        decl = self.parameters()
        for name, d in decl.items():
            t = tensors[name]
            if tuple(t.shape) != tuple(d.shape):
                raise ValueError(f"{type(self).__name__}.{name}: shape {tuple(t.shape)}, expected {d.shape}")
        self.weights = {n: tensors[n] for n in decl}


@dataclass
class NormTail:
    """A small computation on the rows a norm has just produced, which the part after the norm asks it to do in
    the same kernel (the rows are at hand there; a kernel of its own would wait for them and read them back).
    ``kind`` names it; a norm lists the kinds it can do in ``Norm.tails`` and is handed nothing else.
    "router": ``weights`` [E, d], ``k``; the norm fills ``index`` [rows, k] (int32) and ``scores`` [rows, k] (float)
    with each row's k experts and their softmax weights, by the rules of the router kernel."""
    kind: str
    weights: Any = None
    k: int = 0
    index: Any = None
    scores: Any = None


class Norm(Part):
    takes_weighted_rows = False
    can_warm = False           # forward takes ``warm=``: a weight of the next part to fetch into L2 meanwhile
    tails: tuple = ()          # kinds of NormTail that forward(..., tail=) computes along the way

    def forward(self, ctx, x, delta, rows, y) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, ctx, x1, out, cache, state) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def norm_tail(self, ctx, nt: int) -> Optional[NormTail]:
        """What the norm before this part may compute along the way in a step of ``nt`` rows, or None.  If the norm
        lists the kind, it is handed the object and ``forward`` receives it back as ``tail=`` (computed)."""
        return None

    def forward(self, ctx, x1, out):
        """Write the contribution into ``out`` and return None, or return a :class:`WeightedRows`
        that stands for it (``out`` is then left alone)."""
        raise NotImplementedError


class Position(Part):
    def rotation(self):
        """(cos, sin, half_pairing) of a rotary encoding -- float tables [positions, dh/2] on the device and 0
        for adjacent pairs (2i, 2i+1), 1 for halves (i, i + dh/2) -- or None for any other encoding."""
        return None

    def apply(self, ctx, qkv, nh: int, nkvh: int, dh: int) -> None:
        """For an encoding without ``rotation()``: change the step's queries and keys in place.  ``qkv`` is
        [nt, (nh + 2 nkvh) dh] with the heads in the order q, k, v; ``ctx.tok_pos`` holds the positions."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx, x) -> None:
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx, xn, logits) -> None:
        raise NotImplementedError


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Callable] = {}

    def register(self, kind: str, cls=None, *, replace: bool = False):
        def deco(c):
            if kind in self._kinds and not replace:
                raise ValueError(f"{self.what} kind {kind!r} is already registered")
            self._kinds[kind] = c
            return c
        return deco(cls) if cls is not None else deco

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str):
        cls = self._kinds.get(kind)
        if cls is None:
            raise ValueError(f"unknown {self.what} kind {kind!r}; registered: {sorted(self._kinds)}")
        return cls

    def build(self, spec, dtype, device):
        return self.get(spec.kind)(spec.get(), dtype, device)

    def kinds(self):
        return sorted(self._kinds)


EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
NORMS = Registry("norm")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
POSITIONS = Registry("position encoding")
ARRANGEMENTS = Registry("block arrangement")     # kind -> class(LayerSpec, dtype, device); see parts/block.py
