"""CUDA graphs and garbage: an engine that is dropped frees its graphs at once; garbage that owns a graph cannot be
collected inside another engine's capture; a step that fails leaves the cache as it was."""
import gc
import weakref

import pytest
import torch

import transformer_b200 as tb
from tiny import CONFIGS, make_folder, random_prompts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return make_folder(tmp_path_factory.mktemp("lifetime"), "A")


def _decode_until_captured(engine, n_seq=2, steps=4):
    cfg, _ = CONFIGS["A"]
    prompts = random_prompts(cfg["vocab_size"], [5, 9, 3][:n_seq], seed=1)
    slots = [engine.open() for _ in prompts]
    engine.step(slots, prompts)
    outs = [engine.step(slots, [[j + 1]] * n_seq).cpu().clone() for j in range(steps)]
    for s in slots:
        engine.close(s)
    return outs


def test_a_dropped_engine_is_freed_without_the_collector(folder):
    was = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        engine = tb.load(folder, dtype="bfloat16", max_tokens=256)
        _decode_until_captured(engine)
        assert engine._graphs, "the decode steps should have been captured"
        graph = weakref.ref(engine._graphs[2][0])
        ref = weakref.ref(engine)
        del engine
        assert ref() is None, "something keeps the engine alive in a reference cycle"
        assert graph() is None, "the engine's CUDA graph outlived it"
    finally:
        if was:
            gc.enable()


class _Knot:
    """Garbage in a reference cycle that owns a captured CUDA graph, as a dropped engine used to be."""

    def __init__(self):
        self.me = self
        self.x = torch.zeros(8, device="cuda")
        self.graph = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.x += 1          # warm-up outside the capture
        torch.cuda.current_stream().wait_stream(s)
        with torch.cuda.graph(self.graph):
            self.x += 1


def test_capturing_while_garbage_owns_graphs(folder):
    """Engine 1 captures and is dropped without a collection; a knot of garbage that owns a graph lies around and is
    kept from the cyclic collector until engine 2 captures.  Inside that capture the test does what the collector
    would do at some allocation: it collects.  Were the knot still there, destroying its graph would invalidate the
    capture and the step would raise; the engine must have freed it before the capture began, and must keep the
    collector off until the capture ends."""
    cfg, _ = CONFIGS["A"]
    old = gc.get_threshold()
    want = _decode_until_captured(tb.load(folder, dtype="bfloat16", max_tokens=256))
    gc.collect()
    gc.set_threshold(1 << 30)          # enabled, but it never runs by itself: the garbage stays until someone collects
    seen = {}
    try:
        first = tb.load(folder, dtype="bfloat16", max_tokens=256)
        _decode_until_captured(first)
        del first
        knot = weakref.ref(_Knot())
        second = tb.load(folder, dtype="bfloat16", max_tokens=256)
        real = second._forward

        def watching(ctx, logits_out=None):
            if torch.cuda.is_current_stream_capturing():
                seen["collector on"] = gc.isenabled()
                seen["knot alive"] = knot() is not None
                gc.collect()
            return real(ctx, logits_out)
        second._forward = watching
        prompts = random_prompts(cfg["vocab_size"], [5, 9], seed=1)
        slots = [second.open() for _ in prompts]
        second.step(slots, prompts)
        got = [second.step(slots, [[1]] * 2).cpu().clone()]          # the first decode step runs eagerly
        assert knot() is not None and not second._graphs, "the knot should still wait for the cyclic collector"
        got.append(second.step(slots, [[2]] * 2).cpu().clone())      # this one captures
        assert second._graphs and gc.isenabled()
        got += [second.step(slots, [[j + 1]] * 2).cpu().clone() for j in (2, 3)]
        for s in slots:
            second.close(s)
        del second._forward
    finally:
        gc.set_threshold(*old)
    assert seen == {"collector on": False, "knot alive": False}, seen
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    second.release()
    assert not second._graphs and second.workspace.nbytes == 0
    again = _decode_until_captured(second)          # a released engine steps and captures again
    for a, b in zip(again, want):
        assert torch.equal(a, b)


@pytest.mark.parametrize("graphs", [False, True])
def test_a_step_that_raises_leaves_the_cache_as_it_was(folder, graphs):
    cfg, _ = CONFIGS["A"]
    engine = tb.load(folder, dtype="float32", max_tokens=256)
    engine.use_graphs = graphs
    prompt = random_prompts(cfg["vocab_size"], [70], seed=3)[0]
    clean = engine.open()
    engine.step([clean], [prompt[:60]])
    want = [engine.step([clean], [[t]]).cpu().clone() for t in prompt[60:]]     # crosses into a second page
    engine.close(clean)

    s = engine.open()
    engine.step([s], [prompt[:60]])

    def broken(*a, **k):
        raise RuntimeError("the forward pass fails")
    got = []
    for i, t in enumerate(prompt[60:]):
        if i in (1, 4, 5):            # before and at the page boundary (position 64 is token index 4)
            engine.staging = broken       # every step, replayed graph or not, asks for its staging buffer
            with pytest.raises(RuntimeError, match="the forward pass fails"):
                engine.step([s], [[t]])
            with pytest.raises(RuntimeError, match="the forward pass fails"):
                engine.step([s], [prompt[:9]], [[0, 8]])        # a prompt-shaped step fails the same way
            del engine.staging
            assert engine.cache.length(s) == 60 + i
            engine.cache.table.check()
        got.append(engine.step([s], [[t]]).cpu().clone())
    engine.close(s)
    engine.cache.table.check()
    assert engine.cache.table.pages.held == 0
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    with pytest.raises(tb.StepError):
        s = engine.open()
        engine.step([s], [[1, 2]], device_tokens=torch.zeros(1, dtype=torch.int32, device="cuda"))
    assert engine.cache.length(s) == 0      # refused before anything was extended
