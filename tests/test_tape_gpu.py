"""Layers replayed from C++ (engine/tape.py) give the bits that layers run from Python give, and really are replayed."""
import pytest
import torch

import transformer_b200 as tb
from transformer_b200.csrc import lib
from tiny import CONFIGS, make_folder, random_prompts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("tape_models")
    return {n: make_folder(tmp, n) for n in CONFIGS}


def _run(engine, cfg):
    prompts = random_prompts(cfg["vocab_size"], [37, 5, 90], seed=3)
    slots = [engine.open() for _ in prompts]
    outs = [engine.step(slots, prompts, [[0, len(p) - 1] for p in prompts]).cpu().clone()]
    for j in range(4):                     # eager decode, then captured and replayed graphs
        outs.append(engine.step(slots, [[j + 1], [j + 2], [j + 3]]).cpu().clone())
    outs.append(engine.step(slots[:2], [[9, 8, 7], [6]], [[2], [0]]).cpu().clone())     # a ragged step from the cache
    for s in slots:
        engine.close(s)
    return outs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "dense"])
def test_replayed_layers_give_the_same_bits(name, dtype, folders, monkeypatch):
    cfg, _ = CONFIGS[name]
    calls = []
    real = lib.tape_replay
    monkeypatch.setattr(lib, "tape_replay", lambda e, m, n: (calls.append(len(e)), real(e, m, n))[1])
    taped = tb.load(folders[name], dtype=dtype, max_tokens=1024)
    assert taped.use_tapes and all(k is not None for k in taped._run_kind)
    got = _run(taped, cfg)
    layers = cfg["num_hidden_layers"]
    # the first layer is handed nothing, the second records what the later ones replay
    assert (len(calls) > 0) == (layers > 2), f"{len(calls)} replays with {layers} layers"
    n_replayed = len(calls)
    plain = tb.load(folders[name], dtype=dtype, max_tokens=1024)
    plain.use_tapes = False
    want = _run(plain, cfg)
    assert len(calls) == n_replayed, "an engine with tapes off must not replay"
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_many_equal_layers_are_one_recording(tmp_path, monkeypatch):
    """Eight layers: two run from Python (the first is handed nothing by a block before it; the second is recorded),
    six are replayed, in as many calls as the library products cut the layer into segments."""
    cfg = dict(CONFIGS["C"][0], num_hidden_layers=8)
    folder = tb.write_random_model(str(tmp_path / "deep"), cfg, seed=1, std=0.1)
    calls = []
    real = lib.tape_replay
    monkeypatch.setattr(lib, "tape_replay", lambda e, m, n: (calls.append(len(e)), real(e, m, n))[1])
    prompt = random_prompts(cfg["vocab_size"], [200], seed=5)[0]
    outs = []
    for tapes in (True, False):
        eng = tb.load(folder, dtype="bfloat16", max_tokens=512)
        eng.use_tapes = tapes
        s = eng.open()
        before, n0 = len(calls), lib.launch_count
        outs.append(eng.step([s], [prompt], [[0, 199]]).cpu())
        if tapes:
            segments = len(calls) - before
            assert segments % 6 == 0 and 6 <= segments <= 18, f"{segments} replay calls for six layers"
            launched_taped = lib.launch_count - n0
        else:
            assert len(calls) == before and lib.launch_count - n0 == launched_taped, "the same launches either way"
    assert torch.equal(outs[0], outs[1])
    # a recorder needs Python to run in every layer: no replay then
    eng.use_tapes = True
    seen = []
    eng.recorder = lambda name, run, t: seen.append(run)
    before = len(calls)
    s = eng.open()
    eng.step([s], [prompt[:50]])
    assert len(calls) == before and sorted(set(seen)) == list(range(8))
