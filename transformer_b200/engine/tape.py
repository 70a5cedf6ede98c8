"""One layer's launches, recorded once per step and replayed for the other layers from C++.

A forward pass calls a handful of launchers per layer.  From Python each call costs some ten microseconds (views of
scratch memory, argument conversion, the call itself): for a prompt of a few hundred tokens, or for the eager
decode step that sizes a CUDA graph, that is more than the device needs.  But layers built from equal parts make the
SAME calls with the same arguments; only the pointers to their own weights, their part of the cache and their
state differ.  So during a step the first run of every kind of layer is recorded (:class:`LayerTape`) and each later
run of that kind is one call into ``tb_tape_replay`` (csrc/tape.cu), which moves the pointers and calls the
launchers directly.  Work that is not a launcher of this package (a library product) cuts the tape into segments
and is repeated from Python with the run's own weight.  The reference's step is one native call as well
(models/llama/cuda/src/infer.rs:94-147).

Only layers whose parts promise ``launches_only`` (all their device work goes through ``csrc.lib`` launchers or is
reported with ``lib.foreign``) are recorded; anything else runs from Python as before.  Replayed and direct
launches are the same launches: the results are equal bit for bit.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..csrc import lib


class LayerTape:
    def __init__(self):
        self.ops: list = []          # ("launch", name, args) | ("mm", a, w, out)
        self.usable = True
        self.result = None           # what the recorded block returned (its pending contribution)
        self._segments = None

    # ---- the recorder's interface (csrc.lib.recording) ---------------------------------------
    def launch(self, name, args) -> None:
        self.ops.append(("launch", name, args))

    def foreign(self, kind, *tensors) -> None:
        if kind == "mm" and len(tensors) == 3:
            self.ops.append(("mm",) + tuple(tensors))
        else:
            self.usable = False      # work this tape cannot repeat

    # ---- replay --------------------------------------------------------------------------------
    def compile(self, tensors0: Sequence[torch.Tensor]) -> None:
        """tensors0: the recorded run's own tensors (weights, cache, state), in the order every run lists them."""
        where = {t.data_ptr(): i for i, t in enumerate(tensors0)}
        segments, calls = [], []
        for op in self.ops:
            if op[0] == "launch":
                calls.append((op[1], op[2]))
                continue
            if calls:
                segments.append(("launches", lib.tape_entries(calls)))
                calls = []
            _, a, w, out = op
            at = where.get(w.data_ptr())
            if at is None or tuple(tensors0[at].shape) != tuple(w.shape):
                self.usable = False          # a product with something that is not one of the layer's own tensors
                return
            segments.append(("mm", a, at, out))
        if calls:
            segments.append(("launches", lib.tape_entries(calls)))
        self._segments = segments

    def replay(self, maps, n_maps: int, tensors: Sequence[torch.Tensor]):
        for seg in self._segments:
            if seg[0] == "launches":
                lib.tape_replay(seg[1], maps, n_maps)
            else:
                _, a, at, out = seg
                torch.mm(a, tensors[at].t(), out=out)
        return self.result


def run_tensors(layer, cache_view, state) -> Optional[List[torch.Tensor]]:
    """The tensors that belong to one run of a layer, in a fixed order: every part's weights, the run's keys and
    values, its state.  None if the run holds something this scheme does not know how to move."""
    out: List[torch.Tensor] = []
    for pname, part in layer.parts().items():
        for wname in sorted(part.weights):
            out.append(part.weights[wname])
    if cache_view is not None:
        k, v = getattr(cache_view, "k", None), getattr(cache_view, "v", None)
        if not (isinstance(k, torch.Tensor) and isinstance(v, torch.Tensor) and type(cache_view).__name__ == "CacheView"):
            return None
        out += [k, v]
    if state is not None:
        out.append(state)
    return out


def moves(tensors0: Sequence[torch.Tensor], tensors: Sequence[torch.Tensor]):
    """(base, size, delta) for every tensor of the recorded run that lies elsewhere in this run."""
    out = []
    for a, b in zip(tensors0, tensors):
        if tuple(a.shape) != tuple(b.shape) or a.dtype != b.dtype or a.stride() != b.stride():
            return None
        d = b.data_ptr() - a.data_ptr()
        if d:
            out.append((a.data_ptr(), a.numel() * a.element_size(), d))
    return out
