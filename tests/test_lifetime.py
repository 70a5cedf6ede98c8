"""Who keeps whom alive, and what a failed step or a kernel that gave up leaves behind: the parts of these rules
that need no device."""
import gc
import weakref

import pytest
import torch

from transformer_b200.cache.slots import PAGE, CacheError, SequenceTable
from transformer_b200.csrc import lib
from transformer_b200.engine.context import Workspace, weak_callback
from transformer_b200.engine.generate import run_batches


class Owner:
    """Wired like the engine: it owns a workspace and hands it one of its own methods."""

    def __init__(self):
        self.dropped = 0
        self.workspace = Workspace(torch.device("cpu"), on_grow=weak_callback(self.drop))

    def drop(self):
        self.dropped += 1


def test_an_owner_of_a_workspace_is_freed_by_its_reference_count_alone():
    was = gc.isenabled()
    gc.disable()                      # no cyclic collector: only the reference count can free it
    try:
        o = Owner()
        o.workspace.get("a", (4,), torch.float32)
        o.workspace.get("a", (8,), torch.float32)          # grows: the callback reaches the owner
        assert o.dropped == 1
        ws, ref = o.workspace, weakref.ref(o)
        del o
        assert ref() is None, "the workspace keeps its owner alive: a reference cycle"
        ws.get("a", (16,), torch.float32)                  # the owner is gone: the callback does nothing
    finally:
        if was:
            gc.enable()


def test_a_strong_callback_would_have_needed_the_collector():
    """The counter-example, so that the test above cannot pass by accident."""
    class Strong:
        def __init__(self):
            self.workspace = Workspace(torch.device("cpu"), on_grow=self.drop)

        def drop(self):
            pass
    was = gc.isenabled()
    gc.disable()
    try:
        o = Strong()
        ref = weakref.ref(o)
        del o
        assert ref() is not None
    finally:
        if was:
            gc.enable()
    gc.collect()
    assert ref() is None


def test_buffers_kept_at_zero_are_zeroed_again_on_request():
    ws = Workspace(torch.device("cpu"))
    done = ws.get("done", (4,), torch.int32, zero=True)
    other = ws.get("other", (4,), torch.int32)
    done.fill_(3)
    other.fill_(5)
    ws.rezero()
    assert done.tolist() == [0] * 4 and other.tolist() == [5] * 4
    ws.clear()
    assert ws.nbytes == 0


def test_truncate_puts_a_sequence_back_and_loses_no_page():
    t = SequenceTable(max_slots=2, n_pages=5, max_context=1000)
    a, b = t.open(), t.open()
    t.extend(a, 70)                           # two pages
    before = (t.length[a], list(t.page_list[a]), t.pages.free)
    t.extend(a, 100)                          # 170 tokens: three pages
    t.extend(b, 10)
    t.truncate(a, 70)
    assert (t.length[a], t.page_list[a]) == before[:2] and t.pages.free == before[2] - 1
    t.check()
    t.truncate(a, 64)                         # exactly one page left
    assert len(t.page_list[a]) == 1
    t.truncate(a, 0)
    assert t.page_list[a] == [] and t.length[a] == 0
    t.check()
    with pytest.raises(CacheError):
        t.truncate(a, 1)                      # longer than it is
    with pytest.raises(CacheError):
        t.truncate(7, 0)
    t.extend(a, 3 * PAGE)
    t.close(a)
    t.close(b)
    t.check()
    assert t.pages.free == 5 and t.slots.free == 2


def test_a_status_word_that_is_not_zero_raises_after_recovery():
    calls = []
    lib.raise_for_status(0, lambda: calls.append("never"))
    assert calls == []
    for code, what in ((2, "matrix product"), (13, "prompt attention"), (21, "decode attention"), (99, "unknown")):
        with pytest.raises(lib.KernelError, match=what):
            lib.raise_for_status(code, lambda: calls.append(code))
    assert calls == [2, 13, 21, 99]           # what the kernel left behind was put right before the error went up


def test_the_generation_loop_gives_the_slots_back_when_a_kernel_gave_up():
    """collect() raises for a step whose status word is set; the batch's slots are closed all the same and no
    token of that step is kept."""
    held, tokens_seen = set(), []

    def open_slot():
        s = len(held)
        held.add(s)
        return s

    steps = {"n": 0}

    def launch(reqs, slots, toks, n_generated, prev):
        from transformer_b200.engine.generate import Launched
        steps["n"] += 1
        return Launched(list(reqs), steps["n"])

    def collect(step):
        lib.raise_for_status(0 if step.payload < 3 else 12)
        return [7] * len(step.reqs)

    with pytest.raises(lib.KernelError):
        run_batches([[0, 1]], [[1, 2], [3]], [10, 10], frozenset(), 100, open_slot=open_slot,
                    close_slot=held.remove, launch=launch, collect=collect, lookahead=True,
                    on_token=lambda r, t: tokens_seen.append((r, t)))
    assert held == set()
    assert tokens_seen == [(0, 7), (1, 7), (0, 7), (1, 7)]    # two good steps; nothing of the third
