"""The generation loop's decisions, with a fake engine in place of the model (no device)."""
import pytest

from transformer_b200.engine.generate import Timing, plan_batches, verdict
from transformer_b200.sampling import uniform


def test_batches_respect_slots_and_pages():
    lens = [5, 11, 17, 64, 1, 130]
    b = plan_batches(lens, [8] * 6, max_batch=2, n_pages=100, max_context=256)
    assert b == [[0, 1], [2, 3], [4, 5]]
    # pages: requests need 1,1,1,2,1,3 pages (length + 8 new tokens, rounded up to 64)
    b = plan_batches(lens, [8] * 6, max_batch=64, n_pages=4, max_context=256)
    assert b == [[0, 1, 2], [3, 4], [5]]
    assert sorted(i for x in b for i in x) == list(range(6)), "every request exactly once, in order"


def test_batches_refuse_what_can_never_fit():
    with pytest.raises(ValueError, match="exceeds the context"):
        plan_batches([300], [1], max_batch=4, n_pages=100, max_context=256)
    with pytest.raises(ValueError, match="cache pages"):
        plan_batches([200], [1], max_batch=4, n_pages=2, max_context=256)
    with pytest.raises(ValueError, match="empty"):
        plan_batches([0], [1], max_batch=4, n_pages=2, max_context=256)


def test_reach_is_capped_by_the_context():
    # 250 + 100 new tokens would be 350, but the context ends at 256 = 4 pages
    assert plan_batches([250], [100], max_batch=1, n_pages=4, max_context=256) == [[0]]


def test_verdict():
    kw = dict(stop_tokens={2}, max_new=3, max_context=10)
    assert verdict(2, 0, 5, **kw) == (False, "stop")          # the stop token is not kept
    assert verdict(7, 0, 5, **kw) == (True, None)
    assert verdict(7, 2, 5, **kw) == (True, "length")         # the third of three
    assert verdict(7, 0, 10, **kw) == (True, "context")       # sampled, but no room to feed it back
    assert verdict(2, 2, 10, **kw) == (False, "stop")         # stop wins


class FakeEngine:
    """Next token = (last token + 1) % vocab; records every step it is given."""

    def __init__(self, vocab=50, max_context=64, max_slots=3, n_pages=3):
        from transformer_b200.cache.slots import SequenceTable
        self.vocab, self.max_context = vocab, max_context
        self.table = SequenceTable(max_slots, n_pages, max_context)
        self.steps = []

    def step(self, reqs, slots, tokens, n_generated):
        self.steps.append((list(slots), [list(t) for t in tokens]))
        for s, t in zip(slots, tokens):
            self.table.extend(s, len(t))
        return [(t[-1] + 1) % self.vocab for t in tokens]


def _generate(eng, prompts, max_steps, stop_tokens=(0,), lookahead=False):
    from transformer_b200.engine import run_batches
    from transformer_b200.engine.generate import Launched
    limit = [1 << 60 if max_steps is None else max_steps for _ in prompts]
    batches = plan_batches([len(p) for p in prompts], limit, max_batch=eng.table.max_slots,
                           n_pages=eng.table.pages.free, max_context=eng.max_context)
    how = dict(step_and_sample=eng.step)
    if lookahead:
        # a stepper in two halves; "the tokens of the step before, on the device" are the last step's answer
        def launch(reqs, slots, toks, n_generated, prev):
            if toks is None:
                toks = [[prev.payload[prev.reqs.index(r)]] for r in reqs]
            return Launched(list(reqs), eng.step(reqs, slots, toks, n_generated))
        how = dict(launch=launch, collect=lambda step: step.payload, lookahead=True)
    out, why, timing = run_batches(batches, prompts, limit, frozenset(stop_tokens), eng.max_context,
                                   open_slot=eng.table.open, close_slot=eng.table.close, **how)
    from types import SimpleNamespace
    return SimpleNamespace(tokens=out, finished=why, timing=timing, batches=batches)


def test_loop_batches_stops_and_reuses_slots():
    eng = FakeEngine()
    prompts = [[10], [47, 48], [5, 6, 7], [20], [30, 31]]       # 47,48 -> 49 -> 0 = stop
    res = _generate(eng, prompts, max_steps=4)
    assert res.tokens == [[11, 12, 13, 14], [49], [8, 9, 10, 11], [21, 22, 23, 24], [32, 33, 34, 35]]
    assert res.finished == ["length", "stop", "length", "length", "length"]
    assert res.batches == [[0, 1, 2], [3, 4]]                    # three slots, five requests
    # first step of a batch: the prompts, whole and unequal; then one token each
    assert eng.steps[0][1] == [[10], [47, 48], [5, 6, 7]]
    assert eng.steps[1][1] == [[11], [49], [8]]
    assert eng.steps[2][1] == [[12], [9]], "the sequence that stopped left the batch"
    assert eng.table.slots.free == 3 and eng.table.pages.free == 3, "everything was given back"
    eng.table.check()
    assert res.timing.prefill_tokens == 6 + 3 and res.timing.decode_tokens == (3 + 2 + 2) + (2 + 2 + 2)


def test_looking_ahead_gives_the_same_tokens():
    """The next step is launched before the last one's tokens are seen: same tokens, same reasons, and a
    sequence that sampled its stop token has been stepped once more (that token is dropped)."""
    prompts = [[10], [47, 48], [5, 6, 7], [20], [30, 31], [48], [49]]
    for max_steps in (1, 2, 4, 7):
        a = _generate(FakeEngine(), prompts, max_steps=max_steps)
        eng = FakeEngine()
        b = _generate(eng, prompts, max_steps=max_steps, lookahead=True)
        assert (a.tokens, a.finished, a.batches) == (b.tokens, b.finished, b.batches), max_steps
        assert a.timing.prefill_tokens == b.timing.prefill_tokens and a.timing.decode_tokens == b.timing.decode_tokens
        assert eng.table.slots.free == 3 and eng.table.pages.free == 3
        eng.table.check()
    eng = FakeEngine()
    res = _generate(eng, [[10], [47, 48], [5, 6, 7]], max_steps=4, lookahead=True)
    assert res.tokens == [[11, 12, 13, 14], [49], [8, 9, 10, 11]]
    assert eng.steps[1][1] == [[11], [49], [8]]
    assert eng.steps[2][1] == [[12], [0], [9]], "launched before the stop token was seen"
    assert eng.steps[3][1] == [[13], [10]], "then the sequence has left"
    assert len(eng.steps) == 4, "no step is launched for sequences that end by their length"
    # the context ends a sequence without a step too many: one more would not fit the cache
    eng = FakeEngine(max_context=8, n_pages=1, max_slots=1)
    res = _generate(eng, [[1, 2, 3, 4, 5, 6]], max_steps=None, stop_tokens=(), lookahead=True)
    assert res.tokens == [[7, 8, 9]] and res.finished == ["context"] and len(eng.steps) == 3


def test_loop_stops_at_the_context():
    eng = FakeEngine(max_context=8, n_pages=1, max_slots=1)
    res = _generate(eng, [[1, 2, 3, 4, 5, 6]], max_steps=None, stop_tokens=())
    assert res.tokens == [[7, 8, 9]] and res.finished == ["context"]
    assert eng.table.length == {} and eng.table.pages.free == 1


def test_slots_come_back_after_an_error():
    eng = FakeEngine()
    boom = eng.step

    def bad(reqs, slots, tokens, n):
        if len(eng.steps) == 1:
            raise RuntimeError("boom")
        return boom(reqs, slots, tokens, n)
    eng.step = bad
    with pytest.raises(RuntimeError):
        _generate(eng, [[1], [2]], max_steps=5)
    assert eng.table.slots.free == 3


def test_uniform_is_a_function_of_its_arguments():
    a = [uniform(4, r, j) for r in range(3) for j in range(5)]
    assert a == [uniform(4, r, j) for r in range(3) for j in range(5)]
    assert len(set(a)) == len(a) and all(0.0 <= x < 1.0 for x in a)
    assert uniform(5, 0, 0) != uniform(4, 0, 0)
    xs = [uniform(1, 0, j) for j in range(4000)]
    assert abs(sum(xs) / len(xs) - 0.5) < 0.02


def test_timing_table_has_the_references_rows():
    t = Timing(10, 0.5, 30, 1.5)
    text = t.table()
    for word in ("total", "prefill", "decode", "num tokens", "elapse", "time per token"):
        assert word in text
