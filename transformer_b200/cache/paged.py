"""The cache on the device: keys and values in pages, and fixed-size state per sequence.

The reference gives every request one tensor [buf, nblk, 2, nkvh, dh] that the caller owns
(models/llama/common/src/lib.rs:98-107, args.rs:19-25) and sizes it by the context length or half
the free memory (models/llama/cuda/src/infer.rs:74-79).  Here one pool serves all sequences:

* a **slot** per live sequence (its length, its list of pages, its row in every state tensor);
* **pages** of 64 tokens; a sequence holds ceil(length / 64) of them, so the pool is sized by the
  most tokens that live sequences hold, each rounded up to 64;
* **groups**: runs of the model whose mixers need the same kind of storage (kind, heads, head
  size, the kind's own parameters) share one storage object; another need gets a group of its own.
  The storage class is looked up by the need's ``kind`` in :data:`CACHE_KINDS`.  Kind "full" keeps
  keys and values of every position in one pair of tensors K, V [runs, pages, nkvh, 64, dh]; page
  numbers are common to the groups of kind "full".  Another kind (a window of the last W tokens, a
  compressed cache) is a class registered under another name: see :class:`CacheStorage`;
* **state**: for each run whose mixer asks for it, a tensor [slots, *shape], zeroed when a slot
  is opened.

Slots and pages are given back by :meth:`close` and used again by later sequences.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, Registry, StateNeed
from .slots import PAGE, CacheError, SequenceTable

CACHE_KINDS = Registry("cache")     # CacheNeed.kind -> storage class


@dataclass
class CacheView:
    """What one run of a mixer sees of the cache."""
    k: torch.Tensor          # [pages, nkvh, PAGE, dh]
    v: torch.Tensor
    writable: bool           # False when the run reads the cache another run wrote
    kind: str = "full"


class CacheStorage:
    """What a storage class must offer.  One object serves all runs with the same :class:`CacheNeed`.

    ``__init__(need, runs, *, n_pages, max_slots, max_context, dtype, device)``: allocate for ``len(runs)`` runs;
    ``n_pages`` pages of 64 tokens are what the cache's common page pool holds, ``max_slots`` the sequences that
    can be live.  ``view(i, writable)``: what the i-th of these runs hands its mixer as ``cache`` (any object;
    ``writable`` is False for a run that reads another run's cache).  ``open(slot)`` / ``close(slot)``: a
    sequence starts or ends in this slot (storage addressed by slot, not by pages, puts itself in order here)."""

    def __init__(self, need: CacheNeed, runs: List[int], *, n_pages: int, max_slots: int, max_context: int,
                 dtype, device):
        self.need = need
        self.runs = runs

    def view(self, index: int, writable: bool):
        raise NotImplementedError

    def open(self, slot: int) -> None:
        pass

    def close(self, slot: int) -> None:
        pass

    @property
    def nbytes(self) -> int:
        return 0


@CACHE_KINDS.register("full")
class CacheGroup(CacheStorage):
    """Keys and values of every position, in the pages of the common pool."""

    def __init__(self, need: CacheNeed, runs: List[int], *, n_pages: int, max_slots: int, max_context: int,
                 dtype, device):
        super().__init__(need, runs, n_pages=n_pages, max_slots=max_slots, max_context=max_context, dtype=dtype,
                         device=device)
        shape = (len(runs), n_pages, need.nkvh, PAGE, need.dh)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)

    def view(self, index: int, writable: bool) -> CacheView:
        return CacheView(self.k[index], self.v[index], writable=writable, kind=self.need.kind)

    @property
    def nbytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class Cache:
    def __init__(self, cache_needs: Sequence[Optional[CacheNeed]], state_needs: Sequence[Optional[StateNeed]],
                 reads_from: Sequence[Optional[int]], *, max_tokens: int, max_context: int,
                 max_slots: Optional[int], dtype: torch.dtype, device: torch.device):
        """cache_needs[r] / state_needs[r]: what run r's mixer asks for; reads_from[r]: the run whose
        cache run r reads instead of owning one."""
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        n_pages = (max_tokens + PAGE - 1) // PAGE
        if max_slots is None:
            max_slots = min(n_pages, 1024)
        self.table = SequenceTable(max_slots, n_pages, max_context)
        self.dtype = dtype
        self.device = device
        self.groups: List[CacheStorage] = []
        self._where: Dict[int, Tuple[int, int]] = {}     # run -> (group, index in group)
        self._reads_from = list(reads_from)
        by_need: Dict[CacheNeed, List[int]] = {}
        for r, need in enumerate(cache_needs):
            if need is None or reads_from[r] is not None:
                continue
            by_need.setdefault(need, []).append(r)
        for need, runs in by_need.items():
            try:
                storage_cls = CACHE_KINDS.get(need.kind)
            except ValueError as e:
                raise CacheError(str(e)) from None
            g = storage_cls(need, runs, n_pages=n_pages, max_slots=max_slots, max_context=max_context, dtype=dtype,
                            device=device)
            for i, r in enumerate(runs):
                self._where[r] = (len(self.groups), i)
            self.groups.append(g)
        for r, src in enumerate(reads_from):
            if src is not None and cache_needs[r] is not None:
                if src not in self._where:
                    raise CacheError(f"run {r} reads the cache of run {src}, which owns none")
                if cache_needs[src] != cache_needs[r]:
                    raise CacheError(f"run {r} reads the cache of run {src}, but they need different storage")
        self.state: Dict[int, torch.Tensor] = {}
        for r, need in enumerate(state_needs):
            if need is not None:
                self.state[r] = torch.zeros((max_slots, *need.shape), dtype=need.dtype, device=device)

    # ---- sequences ------------------------------------------------------------------------
    def open(self) -> int:
        slot = self.table.open()
        for t in self.state.values():
            t[slot].zero_()
        for g in self.groups:
            g.open(slot)
        return slot

    def close(self, slot: int) -> None:
        self.table.close(slot)
        for g in self.groups:
            g.close(slot)

    def extend(self, slot: int, new_tokens: int) -> int:
        return self.table.extend(slot, new_tokens)

    def truncate(self, slot: int, length: int) -> None:
        self.table.truncate(slot, length)

    def length(self, slot: int) -> int:
        return self.table.length[slot]

    def pages_of(self, slot: int) -> List[int]:
        return self.table.page_list[slot]

    # ---- what a run sees ----------------------------------------------------------------------
    def view(self, run: int) -> Optional[CacheView]:
        src = self._reads_from[run]
        owner = run if src is None else src
        if owner not in self._where:
            return None
        g, i = self._where[owner]
        return self.groups[g].view(i, src is None)

    def state_of(self, run: int) -> Optional[torch.Tensor]:
        return self.state.get(run)

    @property
    def nbytes(self) -> int:
        return sum(g.nbytes for g in self.groups) + sum(t.numel() * t.element_size() for t in self.state.values())
