"""The generation loop above the step function.

The reference's loop serves one sequence: the whole prompt in the first call, then one token per
call, until the end token is sampled (it is neither kept nor fed back) or ``max_steps`` calls are
made; it then prints a table total / prefill / decode with tokens, time and time per token
(test-utils/src/lib.rs:128-203).  This loop does the same for many requests: it cuts them into
batches that fit the cache, runs each batch's prompts (of unequal lengths) in one step and then
one token per live sequence per step, lets sequences that end leave the batch, gives the batch's
slots back when it ends, and goes on with the next batch.

The decisions (which requests form a batch, which sequences go on) are plain functions of
integers, so they can be tested without a device; the model is reached through three callables.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..cache.slots import PAGE
from ..sampling.args import SampleArgs, uniform


@dataclass
class Timing:
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_seconds: float = 0.0

    def table(self) -> str:
        """The reference's table (test-utils/src/lib.rs:175-202) plus tokens per second."""
        rows = [("total", self.prefill_tokens + self.decode_tokens, self.prefill_seconds + self.decode_seconds),
                ("prefill", self.prefill_tokens, self.prefill_seconds),
                ("decode", self.decode_tokens, self.decode_seconds)]
        out = [f"{'':>8} | {'num tokens':>10} | {'elapse':>10} | {'time per token':>14} | {'tokens/s':>10}"]
        for name, n, s in rows:
            per = f"{s / n * 1e3:.3f}ms" if n else "-"
            rate = f"{n / s:.1f}" if s > 0 else "-"
            out.append(f"{name:>8} | {n:>10} | {s * 1e3:>8.3f}ms | {per:>14} | {rate:>10}")
        return "\n".join(out)


@dataclass
class GenerationResult:
    tokens: List[List[int]]            # generated tokens per request, the stop token not included
    finished: List[str]                # "stop" | "length" | "context" per request
    timing: Timing = field(default_factory=Timing)
    batches: List[List[int]] = field(default_factory=list)


def plan_batches(prompt_lens: Sequence[int], max_new: Sequence[int], *, max_batch: int, n_pages: int,
                 max_context: int) -> List[List[int]]:
    """Requests in their order, cut into batches: at most max_batch sequences, and pages enough for
    every sequence of a batch to reach its longest possible length."""
    batches, cur, cur_pages = [], [], 0
    for i, (n, m) in enumerate(zip(prompt_lens, max_new)):
        if n <= 0:
            raise ValueError(f"request {i} has an empty prompt")
        if n > max_context:
            raise ValueError(f"request {i}: a prompt of {n} tokens exceeds the context of {max_context}")
        reach = min(n + max(m, 0), max_context)
        pages = (reach + PAGE - 1) // PAGE
        if pages > n_pages:
            raise ValueError(f"request {i} needs {pages} cache pages of {PAGE} tokens; the cache has {n_pages}")
        if cur and (len(cur) >= max_batch or cur_pages + pages > n_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += pages
    if cur:
        batches.append(cur)
    return batches


def verdict(token: int, n_generated_before: int, length_before: int, *, stop_tokens, max_new: int,
            max_context: int):
    """What happens to a sequence that has just sampled ``token``: (keep the token?, why it ends or
    None).  length_before counts prompt + generated tokens already in the cache."""
    if token in stop_tokens:
        return False, "stop"                       # test-utils/src/lib.rs:166-168
    if n_generated_before + 1 >= max_new:
        return True, "length"
    if length_before + 1 > max_context:
        return True, "context"                     # no room to feed this token back
    return True, None


@dataclass
class Launched:
    """A step that has been handed to the device: the requests it ran, in order, and whatever the
    stepper needs to fetch their tokens later."""
    reqs: List[int]
    payload: object = None


def run_batches(batches, prompts, limit, stops, max_context, *, open_slot, close_slot,
                step_and_sample=None, launch=None, collect=None, lookahead=False, clock=time.perf_counter,
                on_token=None):
    """The loop itself, reached only through callables so that it runs without a device:
    open_slot() -> slot, close_slot(slot), clock() -> seconds, and the stepper, in one of two forms.

    * ``step_and_sample(requests, slots, token lists, tokens generated so far per request)`` -> one new
      token per request: every step waits for the one before.
    * ``launch(requests, slots, token lists or None, generated so far, previous Launched) -> Launched``
      and ``collect(Launched) -> tokens``.  With ``lookahead`` the next step is launched BEFORE the
      tokens of the last one are fetched (token lists = None: the stepper feeds the previous step's
      tokens on the device), so the device never waits for the host.  Whether a sequence ends by its
      length or by the context is known beforehand; only a stop token is not, so a sequence that samples
      one has been stepped once more already: that step's token is dropped, and it leaves one step late.
    """
    if launch is None:
        if step_and_sample is None:
            raise TypeError("run_batches needs step_and_sample, or launch and collect")
        if lookahead:
            raise ValueError("looking ahead needs launch and collect")

        def launch(reqs, slots, toks, n_generated, prev):
            return Launched(list(reqs), step_and_sample(reqs, slots, toks, n_generated))

        def collect(step):
            return step.payload
    out: List[List[int]] = [[] for _ in prompts]
    why: List[Optional[str]] = [None] * len(prompts)
    timing = Timing()
    for batch in batches:
        slots = {r: open_slot() for r in batch}
        try:
            in_cache = {r: len(prompts[r]) for r in batch}      # tokens in the cache after the step being fetched
            ended = {r: False for r in batch}
            t0 = clock()
            step = launch(list(batch), [slots[r] for r in batch], [list(prompts[r]) for r in batch],
                          [0 for _ in batch], None)
            first = True
            while step is not None:
                nxt = None
                if lookahead:
                    # who goes on unless the token about to be fetched is a stop token
                    go = [r for r in step.reqs if not ended[r] and
                          verdict(-1, len(out[r]), in_cache[r], stop_tokens=(), max_new=limit[r],
                                  max_context=max_context)[1] is None]
                    if go:
                        nxt = launch(go, [slots[r] for r in go], None, [len(out[r]) + 1 for r in go], step)
                ids = collect(step)
                t1 = clock()
                if first:
                    timing.prefill_tokens += sum(len(prompts[r]) for r in step.reqs)
                    timing.prefill_seconds += t1 - t0
                    first = False
                else:
                    timing.decode_tokens += sum(1 for r in step.reqs if not ended[r])
                    timing.decode_seconds += t1 - t0
                t0 = t1
                go_on, feed = [], []
                for r, tok in zip(step.reqs, ids):
                    if ended[r]:
                        continue                   # stepped once more after its stop token: dropped
                    keep, end = verdict(tok, len(out[r]), in_cache[r], stop_tokens=stops, max_new=limit[r],
                                        max_context=max_context)
                    if keep:
                        out[r].append(tok)
                        if on_token is not None:
                            on_token(r, tok)
                    if end is None:
                        go_on.append(r)
                        feed.append([tok])
                    else:
                        why[r] = end
                        ended[r] = True
                    in_cache[r] += 1
                if not lookahead and go_on:
                    nxt = launch(go_on, [slots[r] for r in go_on], feed, [len(out[r]) for r in go_on], None)
                step = nxt
        finally:
            for s in slots.values():   # the batch has ended: what it held is used again
                close_slot(s)
    return out, [w or "length" for w in why], timing


def generate(engine, prompts: Sequence[Sequence[int]], *, max_steps: Optional[int] = None,
             sample_args: SampleArgs = SampleArgs(), stop_tokens: Optional[Sequence[int]] = None,
             seed: int = 0, max_batch: Optional[int] = None, on_token: Optional[Callable] = None,
             lookahead: bool = True) -> GenerationResult:
    """Token ids in, token ids out.

    max_steps: most tokens generated per request (the reference's MAX_STEPS counts model calls,
    each of which yields one token; default: until the context is full).  stop_tokens default to
    the ones the model's configuration declares.  ``seed`` fixes the sampler per request.
    ``lookahead``: launch every step before the tokens of the one before have reached the host (see
    :func:`run_batches`); the tokens are the same either way."""
    import torch
    from ..sampling.sampler import Sampler

    spec = engine.spec
    stops = frozenset(spec.stop_tokens if stop_tokens is None else stop_tokens)
    n_req = len(prompts)
    if max_steps is not None and max_steps <= 0:
        return GenerationResult([[] for _ in prompts], ["length"] * n_req)
    limit = [1 << 60 if max_steps is None else int(max_steps) for _ in prompts]   # None: the context ends it
    table = engine.cache.table
    if max_batch is None:
        max_batch = table.max_slots
    max_batch = min(max_batch, table.max_slots - table.slots.held)
    batches = plan_batches([len(p) for p in prompts], limit, max_batch=max_batch,
                           n_pages=table.pages.free, max_context=spec.max_context)
    sampler = getattr(engine, "_sampler", None)
    if sampler is None:
        sampler = engine._sampler = Sampler(engine.device)

    from ..csrc import lib

    # two pinned buffers (at most two steps are in flight): the step's tokens, and in the last element the word
    # that a kernel sets when it gave up on a bounded wait
    n_land = max(1, table.max_slots)
    pinned = getattr(engine, "_token_landing", None)
    if pinned is None:
        pinned = engine._token_landing = [torch.zeros(n_land + 1, dtype=torch.int32, pin_memory=True)
                                          for _ in range(2)]
    turn = [0]

    def launch(reqs, slots, toks, n_generated, prev):
        if toks is not None:
            logits = engine.step(slots, toks)
        else:
            # the tokens of the step before, straight from the device; picked out if some sequences have left
            fed = prev.payload[0]
            if prev.reqs != reqs:
                at = {r: i for i, r in enumerate(prev.reqs)}
                fed = fed[torch.tensor([at[r] for r in reqs], dtype=torch.long, device=fed.device)]
            logits = engine.step(slots, [[0]] * len(reqs), device_tokens=fed)
        u = None if sample_args.greedy else [uniform(seed, r, n) for r, n in zip(reqs, n_generated)]
        ids, _ = sampler.sample(logits, sample_args, u)
        ids = ids.clone()                        # the sampler's own buffer is overwritten by the next step
        host = pinned[turn[0] % 2]
        turn[0] += 1
        host[:len(reqs)].copy_(ids, non_blocking=True)   # the one device-to-host read of the step (infer.rs:140-146)
        lib.kernel_status_async(host[n_land:])           # and four bytes beside it: did every kernel finish its work?
        done = torch.cuda.Event()
        done.record()
        return Launched(list(reqs), (ids, host, done))

    def collect(step):
        _, host, done = step.payload
        done.synchronize()
        engine.check_kernels(int(host[n_land]))          # raises if a kernel returned early: no token of it is used
        return host[:len(step.reqs)].tolist()

    out, why, timing = run_batches(batches, prompts, limit, stops, spec.max_context, open_slot=engine.open,
                                   close_slot=engine.close, launch=launch, collect=collect, lookahead=lookahead,
                                   on_token=on_token)
    return GenerationResult(out, why, timing, batches)
