"""What one step hands to every part: the batch as device index arrays, and scratch memory.

A step's tokens are concatenated (no padding).  For token i of the step:

    tok_ids[i]   its id            tok_seq[i]   which sequence of the batch it belongs to
    tok_pos[i]   its position in that sequence (cache length before the step + offset)

and per sequence b: ``seq_start[b]`` (index of its first token in the step; seq_start[B] = nt),
``seq_pos0[b]`` (its length before the step), ``slots[b]`` (its cache slot = its row in every
per-sequence state tensor), ``page_table[b, :]`` (its pages).  ``want_rows`` lists the tokens whose
logits are asked for.  All of it travels in ONE pinned host buffer and one copy.

The same numbers are kept on the host (``h_*`` lists) for parts that plan on the host.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Sequence, Tuple

import numpy as np
import torch



@dataclass
class AttentionTiles:
    seq: torch.Tensor
    t0: torch.Tensor
    nq: torch.Tensor
    count: int


def weak_callback(method) -> Callable[[], None]:
    """A plain function that calls the bound method ``method`` for as long as its object lives and does nothing
    afterwards.  An object that hands one of its own methods to something it owns would otherwise keep itself
    alive through that something (a reference cycle), and would be freed only when the cyclic collector next runs:
    at an arbitrary allocation, possibly in the middle of someone else's CUDA graph capture."""
    ref = weakref.WeakMethod(method)

    def call() -> None:
        m = ref()
        if m is not None:
            m()
    return call


class Workspace:
    """Named scratch buffers, kept between steps and grown when a step needs more."""

    def __init__(self, device, on_grow=None):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._kept_zero = set()  # keys of the buffers whose users leave them zeroed
        self.frozen = False     # set while a CUDA graph is being captured
        self.on_grow = on_grow  # called before a buffer is replaced (whoever kept its address must forget it)

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """``zero``: the buffer is zeroed when it is made (and made anew when it grows); its users leave it
        zeroed, as the kernels do that count their finished blocks in such a buffer."""
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"scratch buffer {name!r} would grow while a CUDA graph is captured")
            if buf is not None and self.on_grow is not None:
                self.on_grow()
            buf = (torch.zeros if zero else torch.empty)(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            if zero:
                self._kept_zero.add(key)
        return buf[:n].view(*shape)

    def rezero(self) -> None:
        """Zero again the buffers that their users are trusted to leave zeroed (after a kernel returned early)."""
        for key in self._kept_zero:
            self._bufs[key].zero_()

    def clear(self) -> None:
        self._bufs.clear()
        self._kept_zero.clear()

    @property
    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


class StepContext:
    def __init__(self, engine, slots: Sequence[int], tokens: Sequence[Sequence[int]], pos0: Sequence[int],
                 want_rows: Sequence[int], tile_sizes: Sequence[int], fixed_pages: Optional[int] = None,
                 staging=None):
        self.engine = engine
        self.workspace: Workspace = engine.workspace
        self.device = engine.device
        self.dtype = engine.dtype
        cache = engine.cache
        B = len(slots)
        lens = [len(t) for t in tokens]
        nt = sum(lens)
        self.B, self.nt = B, nt
        self.h_slots = list(slots)
        self.h_lens = lens
        self.h_pos0 = list(pos0)
        self.h_want = list(want_rows)
        self.decode = all(n == 1 for n in lens)
        self.max_len_after = max((p + n for p, n in zip(pos0, lens)), default=0)
        page_lists = [cache.pages_of(s) for s in slots]
        self.max_pages = fixed_pages if fixed_pages is not None else max(1, max(len(p) for p in page_lists))

        # ---- pack everything into one int32 array -------------------------------------------
        seq_start = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(lens, out=seq_start[1:])
        tok_ids = np.fromiter((t for ts in tokens for t in ts), dtype=np.int32, count=nt)
        tok_seq = np.repeat(np.arange(B, dtype=np.int32), lens)
        tok_pos = np.concatenate([np.arange(p, p + n, dtype=np.int32) for p, n in zip(pos0, lens)]) if nt else \
            np.zeros(0, np.int32)
        table = np.zeros((B, self.max_pages), dtype=np.int32)
        for b, pl in enumerate(page_lists):
            table[b, :len(pl)] = pl
        parts = {
            "tok_ids": tok_ids, "tok_seq": tok_seq, "tok_pos": tok_pos, "seq_start": seq_start,
            "seq_pos0": np.asarray(pos0, dtype=np.int32), "slots": np.asarray(slots, dtype=np.int32),
            "want_rows": np.asarray(want_rows, dtype=np.int32), "page_table": table.reshape(-1),
        }
        self._tile_counts = {}
        for tq in tile_sizes:
            ts, t0, nq = [], [], []
            for b in range(B):
                for off in range(0, lens[b], tq):
                    ts.append(b)
                    t0.append(int(seq_start[b]) + off)
                    nq.append(min(tq, lens[b] - off))
            parts[f"tile_seq.{tq}"] = np.asarray(ts, dtype=np.int32)
            parts[f"tile_t0.{tq}"] = np.asarray(t0, dtype=np.int32)
            parts[f"tile_nq.{tq}"] = np.asarray(nq, dtype=np.int32)
            self._tile_counts[tq] = len(ts)
        offsets, total = {}, 0
        for k, v in parts.items():
            offsets[k] = (total, v.size)
            total += (v.size + 3) // 4 * 4     # keep every array 16-byte aligned
        host, dev, event = staging if staging is not None else engine.staging(total)
        event.synchronize()                # the copy that last used this host buffer has finished
        hv = host.numpy()
        for k, v in parts.items():
            o, n = offsets[k]
            hv[o:o + n] = v
        dev[:total].copy_(host[:total], non_blocking=True)
        engine.last_h2d_bytes = total * 4
        event.record()
        self._dev = dev
        self._offsets = offsets
        self._views: Dict[str, torch.Tensor] = {}       # made once per step: every layer asks for the same ones
        self._scratch: Dict[tuple, torch.Tensor] = {}
        self.run_index = -1     # which entry of the run order is executing

    def _view(self, name: str) -> torch.Tensor:
        v = self._views.get(name)
        if v is None:
            o, n = self._offsets[name]
            v = self._views[name] = self._dev[o:o + n]
        return v

    tok_ids = property(lambda self: self._view("tok_ids"))
    tok_seq = property(lambda self: self._view("tok_seq"))
    tok_pos = property(lambda self: self._view("tok_pos"))
    seq_start = property(lambda self: self._view("seq_start"))
    seq_pos0 = property(lambda self: self._view("seq_pos0"))
    slots = property(lambda self: self._view("slots"))
    want_rows = property(lambda self: self._view("want_rows"))

    def page_table(self, cache_view=None) -> torch.Tensor:
        """[B, max_pages] pages of each sequence, for the storage kind of ``cache_view``."""
        return self._view("page_table")

    def record(self, name: str, tensor: torch.Tensor) -> None:
        """Hand a copy of an intermediate result to the engine's recorder, if one is set (a debugging
        aid: which experts were chosen, what a part produced).  Costs nothing when none is set."""
        rec = self.engine.recorder
        if rec is not None:
            rec(name, self.run_index, tensor.detach().clone())

    def scratch(self, name: str, shape, dtype, zero: bool = False) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        t = self._scratch.get(key)
        if t is None:
            t = self._scratch[key] = self.workspace.get(name, shape, dtype, zero)
        return t

    def tiles(self, tq: int) -> AttentionTiles:
        """Each sequence's new tokens cut into tiles of tq tokens (the sizes the model's mixers
        announced in ``tile_sizes`` are planned with every step)."""
        if tq not in self._tile_counts:
            raise RuntimeError(f"no query tiles of {tq} tokens were planned for this step")
        return AttentionTiles(self._view(f"tile_seq.{tq}"), self._view(f"tile_t0.{tq}"),
                              self._view(f"tile_nq.{tq}"), self._tile_counts[tq])

    def attention_splits(self, tiles: int, nh: int, nkvh: int) -> int:
        """Slices of the key range per block: enough blocks to fill the GPU when the batch is
        small.  A function of the batch shape only, so a captured graph can keep it."""
        group = nh // nkvh
        blocks = tiles * nkvh * ((group + 15) // 16)
        target = 2 * self.engine.sm_count
        if blocks >= target:
            return 1
        return int(max(1, min(32, target // blocks)))

    def identity_rotation(self, dh: int):
        key = dh
        if key not in self.engine._identity_tables:
            n = self.engine.cache.table.max_context
            self.engine._identity_tables[key] = (torch.ones((n, dh // 2), dtype=torch.float32, device=self.device),
                                                 torch.zeros((n, dh // 2), dtype=torch.float32, device=self.device))
        return self.engine._identity_tables[key]
