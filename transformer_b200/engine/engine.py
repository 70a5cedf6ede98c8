"""The model on the device and its one step function.

:class:`Engine` = the parts built from a :class:`~transformer_b200.parts.spec.ModelSpec` + the
weights bound to them + the cache + scratch memory.  :meth:`Engine.step` is the only way tokens
reach the model: generation, trace replay and the benchmarks all call it.

The reference's step is ``LlamaWorker::launch`` (models/llama/common/src/compute.rs:139-366): a
ragged batch of requests {cache, seq_len, out_len, pos}, embeddings in, logits of the last
``out_len`` rows of each request out.  Differences by design: token ids in (the gather is a
kernel), positions come from the cache's own bookkeeping, any rows may be asked for, the logits
are always float, and nothing inside synchronises with the host.
"""
from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.paged import Cache
from ..cache.slots import CacheError
from ..csrc import lib
from ..parts.block import build_layer, resolve
from ..parts.base import EMBEDDINGS, HEADS, NORMS
from ..parts.spec import ModelSpec
from .context import StepContext, Workspace, weak_callback
from .tape import LayerTape, moves, run_tensors


class StepError(ValueError):
    pass


def _pending_signature(pending):
    """What a block is handed by the block before it, as far as it shapes the block's launches: nothing, a tensor,
    or weighted rows -- with the addresses, which are scratch memory and so the same from layer to layer."""
    if pending is None:
        return None
    if isinstance(pending, torch.Tensor):
        return ("t", pending.data_ptr(), tuple(pending.shape))
    return ("w", pending.rows.data_ptr(), pending.index.data_ptr(), pending.weights.data_ptr(), pending.k,
            tuple(pending.rows.shape))


class Engine:
    def __init__(self, spec: ModelSpec, weights: Dict[tuple, torch.Tensor], dtype: torch.dtype,
                 device: torch.device, *, max_tokens: int, max_slots: Optional[int] = None,
                 max_step_tokens: int = 8192):
        if device.type != "cuda":
            raise RuntimeError("transformer_b200 runs on a CUDA device only; there is no CPU path")
        lib.library()   # fail now, loudly, if the kernels cannot be built or loaded
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.max_step_tokens = int(max_step_tokens)
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.embed = EMBEDDINGS.build(spec.embedding, dtype, device)
        self.layers = [build_layer(ls, dtype, device) for ls in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, dtype, device)
        self.head_part = HEADS.build(spec.head, dtype, device)
        self._bind(weights)
        runs = spec.order
        mixers = [self.layers[e.layer].mixer for e in runs]
        self.cache = Cache([m.cache_need() for m in mixers], [m.state_need() for m in mixers],
                           [e.cache_of for e in runs], max_tokens=max_tokens, max_context=spec.max_context,
                           max_slots=max_slots, dtype=dtype, device=device)
        # weak: the workspace must not keep its owner alive (see weak_callback); an engine that goes out of scope
        # is freed at once, by reference count, and its CUDA graphs with it
        self.workspace = Workspace(device, on_grow=weak_callback(self._drop_graphs))
        self._identity_tables = {}
        self.recorder = None    # callable(name, run index, tensor copy) for debugging; see StepContext.record
        self._tile_sizes = sorted({int(t) for m in mixers for t in getattr(m, "tile_sizes", ())})
        self._staging = []
        self._staging_next = 0
        self._staging_dev = None
        # decode steps (one token per sequence) replay a CUDA graph captured per batch size, if every part of the
        # model says that its forward is fit for that (Part.graph_safe); one part that runs Python per step
        # (reads host lists, branches on values) keeps the whole model on eager steps
        self.graph_safe = all(p.graph_safe for p in [self.embed, self.final_norm, self.head_part, *self.layers])
        self.use_graphs = True
        self.graph_max_batch = 256
        # layers of equal parts are recorded once per step and replayed from C++ for the other runs (engine/tape.py)
        self.use_tapes = True
        self._run_kind = []      # per run: a key that equal runs share, or None if the run cannot be replayed
        self._run_tensors = []   # per run: its own tensors (weights, cache, state)
        self._tape_maps = {}     # (recorded run, run) -> (TapeMap array, count)
        for r, e in enumerate(runs):
            layer = self.layers[e.layer]
            tensors = run_tensors(layer, self.cache.view(r), self.cache.state_of(r)) \
                if getattr(layer, "launches_only", False) else None
            self._run_tensors.append(tensors)
            self._run_kind.append(None if tensors is None else (spec.layers[e.layer], e.cache_of is None))
        self._graphs = {}        # batch size -> (graph, static logits)
        self._graph_seen = {}    # batch size -> decode steps run eagerly so far

    # ---- construction ---------------------------------------------------------------------
    def _bind(self, weights) -> None:
        self.embed.bind({n: weights[("embedding", n)] for n in self.embed.parameters()})
        self.head_part.bind({n: weights[("head", n)] for n in self.head_part.parameters()})
        for i, layer in enumerate(self.layers):
            for pname, part in layer.parts().items():
                part.bind({n: weights[("layers", i, pname, n)] for n in part.parameters()})
        self.final_norm.bind({n: weights[("final_norm", n)] for n in self.final_norm.parameters()})

    @property
    def embedding(self) -> torch.Tensor:
        """The embedding part's table (for a look at the weights; the engine itself goes through the part)."""
        return self.embed.weights["table"]

    @property
    def head(self) -> torch.Tensor:
        return self.head_part.weights["weight"]

    def _graphs_on(self, B: int) -> bool:
        return self.use_graphs and self.graph_safe and B <= self.graph_max_batch

    def _drop_graphs(self) -> None:
        """Captured graphs hold raw addresses of scratch and staging memory; when either moves, they go."""
        if self._graphs:
            torch.cuda.synchronize(self.device)
        self._graphs.clear()
        self._graph_seen.clear()

    def release(self) -> None:
        """Give up the captured graphs and the scratch memory now (the weights and the cache go when the last
        reference to the engine goes).  Call it outside any CUDA graph capture; the engine can still step
        afterwards and captures again.  An engine that is simply dropped does the same through its reference
        count: nothing of it waits for Python's cyclic collector."""
        self._drop_graphs()
        self.workspace.clear()
        self._identity_tables.clear()

    def check_kernels(self, code: Optional[int] = None) -> None:
        """Raise :class:`~transformer_b200.csrc.lib.KernelError` if a kernel with bounded waits gave up since the
        last check (such a kernel returns early and leaves a half-written result).  ``code``: the status word if
        the caller has fetched it already (``lib.kernel_status_async``); else it is read now, which waits for
        the device.  Before raising, the counters that the kernels are trusted to leave at zero are zeroed again,
        so the steps after the error are sound."""
        if code is None:
            code = lib.gemm_tc_status()
        lib.raise_for_status(code, self._after_gave_up)

    def _after_gave_up(self) -> None:
        torch.cuda.synchronize(self.device)
        lib.gemm_tc_status()          # clears the word
        self.workspace.rezero()

    def staging(self, n_ints: int):
        """A pinned host buffer, the device buffer it is copied to, and the event of its last copy."""
        size = max(1 << 16, 1 << (int(n_ints) - 1).bit_length())
        if not self._staging or self._staging[0][0].numel() < size:
            torch.cuda.synchronize(self.device)
            self._drop_graphs()           # captured graphs read the old device buffer
            self._staging = [(torch.empty(size, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                             for _ in range(4)]
            self._staging_dev = torch.empty(size, dtype=torch.int32, device=self.device)
        host, event = self._staging[self._staging_next]
        self._staging_next = (self._staging_next + 1) % len(self._staging)
        return host, self._staging_dev, event

    # ---- sequences ------------------------------------------------------------------------
    def open(self) -> int:
        """A slot for a new sequence."""
        return self.cache.open()

    def close(self, slot: int) -> None:
        """Give back what the sequence holds."""
        self.cache.close(slot)

    # ---- the step ---------------------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None, *, device_tokens: Optional[torch.Tensor] = None
             ) -> torch.Tensor:
        """Run the given next tokens of the given sequences as one batch, from the cache.

        slots[b]: an open slot; tokens[b]: its next tokens (one or many, lengths may differ);
        want[b]: indices into tokens[b] whose logits are wanted (default: the last).  Returns float
        logits [sum of len(want[b]), vocab] on the device, in the order of the batch and of ``want``.

        device_tokens: for one-token steps, an int32 device tensor [B] that holds the tokens (for
        instance what the sampler just wrote); ``tokens`` then only gives the shape.  Nothing comes
        back to the host between such steps.

        The logits of a one-token step may lie in memory that the next such step of the same batch size writes
        again (a replayed CUDA graph has one fixed output): use or copy them before stepping on.  A step that
        raises leaves the sequences as they were before it.
        """
        B = len(slots)
        if len(tokens) != B:
            raise StepError(f"{B} slots but {len(tokens)} token lists")
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        if len(want) != B:
            raise StepError(f"{B} slots but {len(want)} want lists")
        if len(set(slots)) != B:
            raise StepError("a slot appears twice in one step")
        V = self.spec.vocab
        for b in range(B):
            n = len(tokens[b])
            if n == 0:
                raise StepError(f"sequence {b} of the step brings no token")
            for t in tokens[b]:
                if not (0 <= int(t) < V):
                    raise StepError(f"token {t} lies outside the vocabulary of {V}")
            for w in want[b]:
                if not (0 <= int(w) < n):
                    raise StepError(f"wanted place {w} lies outside the {n} tokens of sequence {b}")
        n_total = sum(len(t) for t in tokens)
        one_each = n_total == B and all(list(w) == [0] for w in want)
        if device_tokens is not None and not one_each:
            raise StepError("device_tokens serve steps of one token per sequence that want its logits")
        # room for everything first: a step either runs whole or not at all
        need = sum(self.cache.table.pages_needed(s, len(t)) for s, t in zip(slots, tokens))
        if need > self.cache.table.pages.free:
            raise CacheError(f"cache full: the step needs {need} more pages, {self.cache.table.pages.free} are free")
        for s, t in zip(slots, tokens):
            if self.cache.length(s) + len(t) > self.spec.max_context:
                raise CacheError(f"slot {s} would exceed the context of {self.spec.max_context}")
        before = [self.cache.length(s) for s in slots]
        try:
            pos0 = [self.cache.extend(s, len(t)) for s, t in zip(slots, tokens)]
            if one_each and (device_tokens is not None or self._graphs_on(B)):
                return self._run_decode(slots, tokens, pos0, device_tokens)
            if n_total <= self.max_step_tokens:
                rows, base = [], 0
                for b in range(B):
                    rows.extend(base + int(w) for w in want[b])
                    base += len(tokens[b])
                return self._run(slots, tokens, pos0, rows)
            return self._run_in_pieces(slots, tokens, pos0, want)
        except BaseException:
            # nothing of a failed step stays: the sequences are as long as before it, their new pages are free
            for s, n in zip(slots, before):
                if self.cache.length(s) > n:
                    self.cache.truncate(s, n)
            raise

    def _run_in_pieces(self, slots, tokens, pos0, want) -> torch.Tensor:
        """A step larger than the scratch memory allows runs as consecutive pieces of the token
        axis; a sequence cut by a piece boundary continues from the cache in the next piece."""
        n_want = sum(len(w) for w in want)
        out = torch.empty((n_want, self.spec.vocab), dtype=torch.float32, device=self.device)
        # where each wanted row goes in `out`
        order, k = {}, 0
        for b in range(len(slots)):
            for w in want[b]:
                order.setdefault((b, int(w)), []).append(k)
                k += 1
        cur = [0] * len(slots)
        b = 0
        while b < len(slots):
            p_slots, p_tokens, p_pos0, p_rows, p_dest, room, base = [], [], [], [], [], self.max_step_tokens, 0
            while b < len(slots) and room > 0:
                take = min(room, len(tokens[b]) - cur[b])
                lo, hi = cur[b], cur[b] + take
                p_slots.append(slots[b])
                p_tokens.append(tokens[b][lo:hi])
                p_pos0.append(pos0[b] + lo)
                for i in range(lo, hi):
                    for dest in order.get((b, i), ()):
                        p_rows.append(base + i - lo)
                        p_dest.append(dest)
                base += take
                room -= take
                cur[b] = hi
                if hi == len(tokens[b]):
                    b += 1
            logits = self._run(p_slots, p_tokens, p_pos0, p_rows)
            if p_dest:
                out[torch.tensor(p_dest, device=self.device)] = logits
        return out

    def _run_decode(self, slots, tokens, pos0, device_tokens=None) -> torch.Tensor:
        """One token for each of B sequences.  The first such step of a batch size runs eagerly
        (it also sizes the scratch memory), the second is captured into a CUDA graph, and from then
        on the step is: copy the step's index arrays, replay.  The arrays have the same layout at
        every step of a batch size (the page table has its full width), so the graph stays valid."""
        B = len(slots)
        fixed = self.cache.table.max_pages_per_seq
        ctx = StepContext(self, slots, tokens, pos0, list(range(B)), self._tile_sizes, fixed_pages=fixed)
        if device_tokens is not None:
            ctx.tok_ids.copy_(device_tokens.view(-1)[:B])
        if not self._graphs_on(B):
            return self._forward(ctx)
        entry = self._graphs.get(B)
        if entry is None:
            seen = self._graph_seen.get(B, 0)
            self._graph_seen[B] = seen + 1
            if seen == 0:
                return self._forward(ctx)
            logits = torch.empty((B, self.spec.vocab), dtype=torch.float32, device=self.device)
            graph = torch.cuda.CUDAGraph()
            before = lib.launch_count
            self.workspace.frozen = True      # scratch must not move while it is being captured
            # Nothing may destroy a CUDA graph while this one is captured (that invalidates the capture).  Python
            # frees garbage that sits in reference cycles at arbitrary allocations, and such garbage may own graphs
            # (another engine, anything of torch's): free it now, and keep the collector off until the capture ends.
            gc.collect()
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    self._forward(ctx, logits)
            finally:
                if collecting:
                    gc.enable()
                self.workspace.frozen = False
            entry = (graph, logits, lib.launch_count - before)
            lib.launch_count = before
            self._graphs[B] = entry
        graph, logits, nodes = entry
        graph.replay()
        lib.launch_count += nodes             # a replay launches every captured kernel again
        return logits

    def _run(self, slots, tokens, pos0, rows, *, fixed_pages=None, logits_out=None) -> torch.Tensor:
        ctx = StepContext(self, slots, tokens, pos0, rows, self._tile_sizes, fixed_pages=fixed_pages)
        return self._forward(ctx, logits_out)

    def _maps_between(self, r0: int, r: int):
        key = (r0, r)
        if key not in self._tape_maps:
            mv = moves(self._run_tensors[r0], self._run_tensors[r])
            self._tape_maps[key] = None if mv is None else (lib.tape_maps(mv), len(mv))
        return self._tape_maps[key]

    def _forward(self, ctx: StepContext, logits_out=None) -> torch.Tensor:
        with lib.stream_scope():       # also inside a capture: the scope then holds the capturing stream
            return self._forward_on_stream(ctx, logits_out)

    def _forward_on_stream(self, ctx: StepContext, logits_out=None) -> torch.Tensor:
        nt, d, V = ctx.nt, self.spec.width, self.spec.vocab
        x = ctx.scratch("stream", (nt, d), torch.float32)
        self.embed.forward(ctx, x)
        pending = None
        taping = self.use_tapes and self.recorder is None
        tapes = {}                  # kind of run and of what it is handed -> (recorded run, its tape)
        for r, entry in enumerate(self.spec.order):
            layer = self.layers[entry.layer]
            ctx.run_index = r
            kind = self._run_kind[r] if taping else None
            if kind is None:
                pending = layer.forward(ctx, x, pending, self.cache.view(r), self.cache.state_of(r))
                continue
            kind = (kind, _pending_signature(pending))
            known = tapes.get(kind)
            if known is None:
                tape = LayerTape()
                with lib.recording(tape):
                    pending = layer.forward(ctx, x, pending, self.cache.view(r), self.cache.state_of(r))
                tape.result = pending
                tapes[kind] = (r, tape)
                continue
            r0, tape = known
            if tape.usable and tape._segments is None:
                tape.compile(self._run_tensors[r0])
            maps = self._maps_between(r0, r) if tape.usable else None
            if maps is None:
                pending = layer.forward(ctx, x, pending, self.cache.view(r), self.cache.state_of(r))
            else:
                pending = tape.replay(maps[0], maps[1], self._run_tensors[r])
        n_out = len(ctx.h_want)
        logits = logits_out if logits_out is not None else \
            torch.empty((n_out, V), dtype=torch.float32, device=self.device)
        if n_out:
            xn = ctx.scratch("final.xn", (n_out, d), self.dtype)
            pending = resolve(pending, self.final_norm, ctx.scratch("block.delta", (nt, d), self.dtype))
            self.final_norm.forward(ctx, x, pending, ctx.want_rows, xn)
            self.head_part.forward(ctx, xn, logits)
        return logits
