"""The model as data: which parts make up each layer, and the order in which layers run.

Nothing here computes.  An architecture's ``build_spec`` turns a typed configuration into a
:class:`ModelSpec`; the engine builds parts from it through the part registries and never asks
which architecture it came from.

* A :class:`PartSpec` is a registered kind (``"attention"``, ``"moe"``, ``"rmsnorm"``, ...) with
  its sizes and constants as parameters.
* A :class:`LayerSpec` names the parts of one layer and their arrangement in the block.  Layers may
  differ from one another: each carries its own mixer and feed-forward spec.
* ``ModelSpec.order`` is the run order: a list of :class:`RunEntry`.  It may name a layer twice
  (weights shared, each run with a cache entry of its own unless told otherwise) or let a run read
  the cache that another run wrote (``cache_of``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def of(kind: str, **params) -> "PartSpec":
        return PartSpec(kind, tuple(sorted(params.items())))

    def get(self) -> Dict[str, Any]:
        return dict(self.params)


@dataclass(frozen=True)
class LayerSpec:
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: Optional[PartSpec] = None          # an arrangement says which of these it needs
    feed_forward_norm: Optional[PartSpec] = None
    arrangement: str = "pre_norm"   # a registered kind; pre_norm: x += mixer(norm(x)); x += ff(norm(x))  (compute.rs:204-336)
    extra: Tuple[Tuple[str, PartSpec], ...] = ()   # further parts by name, for arrangements that have them


@dataclass(frozen=True)
class RunEntry:
    layer: int                      # index into ModelSpec.layers
    cache_of: Optional[int] = None  # index into ModelSpec.order whose cache this run reads and does not write


@dataclass(frozen=True)
class ModelSpec:
    width: int
    vocab: int
    max_context: int
    layers: Tuple[LayerSpec, ...]
    order: Tuple[RunEntry, ...]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    stop_tokens: Tuple[int, ...] = ()

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for i, e in enumerate(self.order):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"run entry {i} names layer {e.layer}, but there are {len(self.layers)}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"run entry {i} reads the cache of entry {e.cache_of}, which must come earlier")
                if self.order[e.cache_of].cache_of is not None:
                    raise ValueError(f"run entry {i} reads the cache of entry {e.cache_of}, which owns none")
