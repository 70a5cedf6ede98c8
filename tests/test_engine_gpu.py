"""The engine through its Python API: long decoding, first tokens, slots used again, steps cut
into pieces, CUDA-graph steps, errors, and generation through the entry point."""
import json
import os
import subprocess
import sys

import pytest
import torch

import transformer_b200 as tb
from plain import llama_moe_plain as P
from tiny import (BF16_REL_TOL, CONFIGS, FP32_TOL, ROOT, check_generation, check_request, make_folder, n_moe_layers,
                  random_prompts)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("engine_models")
    return {n: make_folder(tmp, n) for n in CONFIGS}


class Recorder:
    """Collects the experts chosen per run of the model for the steps it watches."""

    def __init__(self, engine):
        self.engine, self.items = engine, []
        engine.recorder = self

    def __call__(self, name, run, t):
        if name == "moe.topk_idx":
            self.items.append(t.cpu())

    def take(self):
        out, self.items = self.items, []
        return out           # [runs] of [nt, k]


def _run_and_check(engine, cfg, tensors, dtype, tokens, cuts, label):
    """Feed ``tokens`` of one request in consecutive pieces of the given lengths and compare every
    position with the plain implementation."""
    rec = Recorder(engine)
    engine.use_graphs = False      # the recorder needs Python to run; graphs are compared separately
    slot = engine.open()
    got, routes, pos = {}, {}, 0
    try:
        for n in cuts:
            piece = tokens[pos:pos + n]
            lg = engine.step([slot], [piece], [list(range(n))]).cpu()
            r = rec.take()
            for i in range(n):
                got[pos + i] = lg[i]
                if r:
                    routes[pos + i] = torch.stack([x[i] for x in r])
            pos += n
    finally:
        engine.close(slot)
        engine.recorder = None
        engine.use_graphs = True
    rt = None
    if n_moe_layers(cfg):
        rt = torch.stack([routes[p] for p in range(len(tokens))], dim=1).numpy()
    return check_request(cfg, tensors, tokens, got, rt, dtype, label)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_to_the_end_of_the_context(name, dtype, folders):
    cfg, _ = CONFIGS[name]
    _, tensors = P.read_folder(folders[name])
    n = cfg["max_position_embeddings"]
    tokens = random_prompts(cfg["vocab_size"], [n], seed=11)[0]
    engine = tb.load(folders[name], dtype=dtype, max_tokens=n + 64)
    _run_and_check(engine, cfg, tensors, dtype, tokens, [5] + [1] * (n - 5), f"long decoding {name}")
    with pytest.raises(tb.CacheError):       # one token more than the context holds
        s = engine.open()
        try:
            engine.step([s], [tokens])
            engine.step([s], [[1]])
        finally:
            engine.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype, folders):
    cfg, _ = CONFIGS["B"]
    _, tensors = P.read_folder(folders["B"])
    engine = tb.load(folders["B"], dtype=dtype, max_tokens=256)
    for cuts in ([1], [1, 1], [1, 1, 1], [2, 1], [3]):
        tokens = random_prompts(cfg["vocab_size"], [sum(cuts)], seed=sum(cuts) + len(cuts))[0]
        _run_and_check(engine, cfg, tensors, dtype, tokens, cuts, f"first tokens {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_slot_used_again_sees_nothing_of_its_past(dtype, folders):
    cfg, _ = CONFIGS["A"]
    _, tensors = P.read_folder(folders["A"])
    engine = tb.load(folders["A"], dtype=dtype, max_tokens=128, max_slots=1)   # one slot, two pages: all reuse
    long, short = random_prompts(cfg["vocab_size"], [128, 40], seed=5)
    _run_and_check(engine, cfg, tensors, dtype, long, [100] + [1] * 28, "first tenant")
    _run_and_check(engine, cfg, tensors, dtype, short, [7, 20] + [1] * 13, "second tenant of the same slot and pages")
    engine.cache.table.check()
    assert engine.cache.table.pages.free == 2 and engine.cache.table.slots.free == 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_cut_into_pieces_changes_nothing(dtype, folders):
    """Config C reaches the tensor-core prompt kernels in bfloat16 (attention with heads of 64, grouped expert
    products): whole against pieces, and both paths against the plain implementation at every wanted place."""
    cfg, _ = CONFIGS["C"]
    _, tensors = P.read_folder(folders["C"])
    prompts = random_prompts(cfg["vocab_size"], [90, 33, 150], seed=8)
    whole = tb.load(folders["C"], dtype=dtype, max_tokens=512)
    pieces = tb.load(folders["C"], dtype=dtype, max_tokens=512, max_step_tokens=64)   # 273 tokens: 5 pieces
    outs = []
    want = [[0, len(p) // 2, len(p) - 1] for p in prompts]
    rec = Recorder(whole)
    for eng in (whole, pieces):
        slots = [eng.open() for _ in prompts]
        outs.append(eng.step(slots, prompts, want).cpu())
        if eng is whole:
            routes = torch.stack(rec.take())             # [layers, 273, k]
            whole.recorder = None
        outs.append(eng.step(slots, [[3], [4], [5]]).cpu())
    tol = 1e-5 if dtype == "float32" else BF16_REL_TOL * float(outs[0].abs().max())
    assert float((outs[0] - outs[2]).abs().max()) <= tol
    assert float((outs[1] - outs[3]).abs().max()) <= tol
    base = 0
    for i, p in enumerate(prompts):
        got = {w: outs[0][3 * i + j] for j, w in enumerate(want[i])}
        check_request(cfg, tensors, p, got, routes[:, base:base + len(p)].numpy(), dtype, f"whole step, request {i}")
        base += len(p)


@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_steps_equal_eager_steps(dtype, folders):
    """Decode steps replay a CUDA graph from their third use on; the logits must not change by a bit,
    for a batch that shrinks and across a page boundary."""
    cfg, _ = CONFIGS["B"]
    prompts = random_prompts(cfg["vocab_size"], [60, 62, 3], seed=9)
    feeds = random_prompts(cfg["vocab_size"], [10, 10, 10], seed=10)
    results = []
    for graphs in (False, True):
        eng = tb.load(folders["B"], dtype=dtype, max_tokens=512)
        eng.use_graphs = graphs
        slots = [eng.open() for _ in prompts]
        eng.step(slots, prompts)
        outs = []
        for j in range(10):
            live = slots if j < 6 else slots[:2]              # the third sequence ends earlier
            outs.append(eng.step(live, [[feeds[i][j]] for i in range(len(live))]).cpu().clone())
        results.append(outs)
        assert bool(eng._graphs) == graphs
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_step_refuses_bad_input_and_changes_nothing(folders):
    eng = tb.load(folders["A"], dtype="float32", max_tokens=128)
    s = eng.open()
    for bad in (lambda: eng.step([s], [[256]]), lambda: eng.step([s], [[-1]]), lambda: eng.step([s], [[]]),
                lambda: eng.step([s], [[1, 2]], [[2]]), lambda: eng.step([s, s], [[1], [2]]),
                lambda: eng.step([s], [[1], [2]])):
        with pytest.raises(tb.StepError):
            bad()
    with pytest.raises(tb.CacheError):
        eng.step([s], [[1] * 129])                 # beyond the context
    s2 = eng.open()
    eng.step([s], [[1] * 100])
    with pytest.raises(tb.CacheError, match="cache full"):
        eng.step([s2], [[1] * 10])                 # 128 tokens of cache: two pages, both taken
    assert eng.cache.length(s) == 100 and eng.cache.length(s2) == 0
    eng.cache.table.check()
    with pytest.raises(tb.CacheError):
        eng.close(99)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "dense"])
def test_greedy_generation_through_the_entry_point(name, dtype, folders):
    cfg, _ = CONFIGS[name]
    _, tensors = P.read_folder(folders[name])
    prompts = random_prompts(cfg["vocab_size"], [5, 11, 17, 1, 30], seed=1)
    engine = tb.load(folders[name], dtype=dtype, max_tokens=256)
    res = tb.generate(engine, prompts, max_steps=8, stop_tokens=(), max_batch=3)     # two batches, slots reused
    assert res.batches == [[0, 1, 2], [3, 4]] and all(len(t) == 8 for t in res.tokens)
    check_generation(engine, cfg, tensors, prompts, res.tokens, res.batches, dtype)
    if dtype == "float32":
        assert res.tokens == [P.greedy_generate(cfg, tensors, p, 8) for p in prompts]
    assert engine.cache.table.slots.held == 0 and engine.cache.table.pages.held == 0


def test_stop_tokens_end_a_sequence_early(folders):
    cfg, _ = CONFIGS["A"]
    _, tensors = P.read_folder(folders["A"])
    prompts = random_prompts(cfg["vocab_size"], [5, 11, 17], seed=1)
    engine = tb.load(folders["A"], dtype="float32", max_tokens=256)
    free = tb.generate(engine, prompts, max_steps=8, stop_tokens=()).tokens
    stop = free[1][3]                                   # the 4th token of the second request
    res = tb.generate(engine, prompts, max_steps=8, stop_tokens=[stop])
    for f, g, why in zip(free, res.tokens, res.finished):
        cut = f.index(stop) if stop in f else len(f)
        assert g == f[:cut] and why == ("stop" if stop in f else "length")
    assert res.finished[1] == "stop" and len(res.tokens[1]) <= 3


@pytest.mark.parametrize("dtype", DTYPES)
def test_published_workloads(dtype, tmp_path):
    """The two tiny workloads as stated (weights N(0, 0.02)): A: prompts 5/11/17, 8 greedy steps;
    B: prompts 1/9/30/64, 12 steps at temperature 0.8 with sampler seed 4."""
    from transformer_b200.sampling import uniform
    fa, fb = make_folder(tmp_path, "A", std=0.02), make_folder(tmp_path, "B", std=0.02)
    (ca, _), (cb, _) = CONFIGS["A"], CONFIGS["B"]
    _, ta = P.read_folder(fa)
    _, tb_ = P.read_folder(fb)
    ea = tb.load(fa, dtype=dtype, max_tokens=256)
    pa = random_prompts(ca["vocab_size"], [5, 11, 17], seed=1)
    res = tb.generate(ea, pa, max_steps=8, stop_tokens=())
    check_generation(ea, ca, ta, pa, res.tokens, res.batches, dtype)
    eb = tb.load(fb, dtype=dtype, max_tokens=512)
    pb = random_prompts(cb["vocab_size"], [1, 9, 30, 64], seed=3)
    args = tb.SampleArgs(temperature=0.8)
    res = tb.generate(eb, pb, max_steps=12, sample_args=args, seed=4, stop_tokens=())
    together = res.tokens
    check_generation(eb, cb, tb_, pb, together, res.batches, dtype,
                     sample=(args, {r: [uniform(4, r, j) for j in range(12)] for r in range(4)}))
    assert together == tb.generate(eb, pb, max_steps=12, sample_args=args, seed=4, stop_tokens=()).tokens, "repeatable"
    assert together != tb.generate(eb, pb, max_steps=12, sample_args=args, seed=5, stop_tokens=()).tokens


def test_command_line(folders):
    env = dict(os.environ, TEST_MODEL=folders["A"], TEMPERATURE="0", MAX_STEPS="5", PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-m", "transformer_b200", "generate", "--prompt", "7 8 9", "--prompt",
                          "1,2", "--dtype", "float32", "--json"], env=env, capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    got = json.loads(out.stdout.strip().splitlines()[-1])
    cfg, tensors = P.read_folder(folders["A"])
    assert got["tokens"] == [P.greedy_generate(cfg, tensors, p, 5) for p in ([7, 8, 9], [1, 2])]
    out = subprocess.run([sys.executable, "-m", "transformer_b200", "inspect", "--model", folders["B"]],
                         env=env, capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0 and "nexp=6" in out.stdout and "architecture: llama" in out.stdout


def test_a_gguf_file_gives_the_same_model(folders, tmp_path):
    """The reference's own container: the same tensors under the same names load to the same logits."""
    pytest.importorskip("gguf")
    from safetensors.torch import load_file
    from test_gguf import write_gguf
    cfg, _ = CONFIGS["A"]
    tensors = load_file(os.path.join(folders["A"], "model.safetensors"))
    path = write_gguf(str(tmp_path / "a.gguf"), cfg, tensors)
    prompt = random_prompts(cfg["vocab_size"], [20], seed=2)[0]
    outs = []
    for src in (folders["A"], path):
        eng = tb.load(src, dtype="float32", max_tokens=128)
        s = eng.open()
        outs.append(eng.step([s], [prompt], [list(range(20))]).cpu())
    assert float((outs[0] - outs[1]).abs().max()) < 2e-5      # epsilon travels as float32 in GGUF metadata


def test_a_step_that_wants_nothing_still_fills_the_cache(folders):
    cfg, _ = CONFIGS["A"]
    _, tensors = P.read_folder(folders["A"])
    eng = tb.load(folders["A"], dtype="float32", max_tokens=128)
    p = random_prompts(cfg["vocab_size"], [12], seed=4)[0]
    s = eng.open()
    out = eng.step([s], [p[:8]], [[]])
    assert tuple(out.shape) == (0, cfg["vocab_size"]) and eng.cache.length(s) == 8
    lg = eng.step([s], [p[8:]], [[0, 3]]).cpu()
    ref = P.forward(cfg, tensors, p, want=[8, 11])
    assert float((lg - ref).abs().max()) <= FP32_TOL


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_wide_decode_batch_equals_its_sequences_alone(dtype, folders):
    """48 sequences of unequal lengths decode together (more than 128 (token, expert) pairs: the experts take the
    prompt kernels with dispatch lists, which the router's last block builds), then each alone (no lists, the
    decode kernels): the same logits within the rounding of the path, whatever else is in the batch.  Where
    rounding tipped a near-tie of the router the other way the logits are not compared; that must stay rare."""
    cfg, _ = CONFIGS["B"]
    n = 48
    lengths = [1 + (7 * i) % 40 for i in range(n)]
    prompts = random_prompts(cfg["vocab_size"], lengths, seed=21)
    feeds = random_prompts(cfg["vocab_size"], [4] * n, seed=22)
    eng = tb.load(folders["B"], dtype=dtype, max_tokens=64 * n, max_slots=n + 1)
    eng.use_graphs = False
    rec = Recorder(eng)
    slots = [eng.open() for _ in range(n)]
    eng.step(slots, prompts)
    rec.take()
    together, chosen = [], []
    for j in range(4):
        together.append(eng.step(slots, [[feeds[i][j]] for i in range(n)]).cpu().clone())
        chosen.append(rec.take())                      # [runs] of [n, k]
    for s in slots:
        eng.close(s)
    compared = tipped = 0
    for i in range(0, n, 5):
        s = eng.open()
        eng.step([s], [prompts[i]])
        rec.take()
        for j in range(4):
            alone = eng.step([s], [[feeds[i][j]]]).cpu()[0]
            mine = rec.take()
            if any(sorted(a[0].tolist()) != sorted(b[i].tolist()) for a, b in zip(mine, chosen[j])):
                tipped += 1
                break                                  # the sequence's cache differs from here on
            tol = FP32_TOL if dtype == "float32" else 2 * BF16_REL_TOL * float(alone.abs().max())
            assert float((together[j][i] - alone).abs().max()) <= tol, f"sequence {i}, step {j}"
            compared += 1
        eng.close(s)
    eng.recorder = None
    eng.cache.table.check()
    assert compared >= 20 and (dtype != "float32" or tipped == 0), (compared, tipped)


@pytest.mark.parametrize("dtype", DTYPES)
def test_looking_ahead_changes_no_token(dtype, folders):
    """`generate` launches each step before the last one's tokens have reached the host.  Same tokens and the same
    reasons to stop as the strict order, greedy and sampled, with stop tokens that really occur (so that sequences
    leave the batch at different times and a step too many is dropped), over two batches (three slots)."""
    cfg, _ = CONFIGS["A"]
    prompts = random_prompts(cfg["vocab_size"], [3, 17, 64, 1, 30, 9, 70], seed=31)
    engine = tb.load(folders["A"], dtype=dtype, max_tokens=1024, max_slots=3)
    for args in (tb.SampleArgs(), tb.SampleArgs(temperature=0.9, top_k=20, top_p=0.95)):
        free = tb.generate(engine, prompts, max_steps=40, stop_tokens=(), sample_args=args, seed=5, lookahead=False)
        # stop tokens that occur: the most frequent tokens of the free run
        flat = [t for seq in free.tokens for t in seq]
        stops = tuple(sorted(set(flat), key=lambda t: -flat.count(t))[:3])
        strict = tb.generate(engine, prompts, max_steps=40, stop_tokens=stops, sample_args=args, seed=5, lookahead=False)
        ahead = tb.generate(engine, prompts, max_steps=40, stop_tokens=stops, sample_args=args, seed=5, lookahead=True)
        assert ahead.tokens == strict.tokens and ahead.finished == strict.finished
        assert "stop" in strict.finished and any(len(t) < 40 for t in strict.tokens)
        assert ahead.timing.decode_tokens == strict.timing.decode_tokens
    engine.cache.table.check()
    assert engine.cache.table.slots.free == 3


# ---------------------------------------------------------------------------------------------
def _decode_batch(engine, prompts, feeds, steps):
    slots = [engine.open() for _ in prompts]
    engine.step(slots, prompts)
    outs = [engine.step(slots, [[f[j]] for f in feeds]).cpu().clone() for j in range(steps)]
    for s in slots:
        engine.close(s)
    return outs


@pytest.mark.parametrize("n", [24, 64])
def test_wide_bfloat16_decode_batches_through_graphs(n, folders):
    """A decode step of 24 or 64 sequences is a captured graph whose dense products (more than 16 rows) are library
    calls.  Without experts (no near-ties to fall either way) every sequence's logits are held against the plain
    implementation and against the sequence alone; with experts the captured steps equal the eager ones bit for
    bit."""
    cfg, _ = CONFIGS["dense"]
    _, tensors = P.read_folder(folders["dense"])
    lengths = [1 + (11 * i) % 60 for i in range(n)]
    prompts = random_prompts(cfg["vocab_size"], lengths, seed=41)
    feeds = random_prompts(cfg["vocab_size"], [5] * n, seed=42)
    eng = tb.load(folders["dense"], dtype="bfloat16", max_tokens=128 * n, max_slots=n + 1)
    together = _decode_batch(eng, prompts, feeds, 5)
    assert n in eng._graphs, "the decode steps of this batch size should have been captured"
    for i in range(0, n, 7):
        alone = _decode_batch(eng, [prompts[i]], [feeds[i]], 5)
        seq = prompts[i] + feeds[i]
        ref = P.forward(cfg, tensors, seq, want=list(range(len(prompts[i]), len(seq))))
        tol = BF16_REL_TOL * float(ref.abs().max())
        for j in range(5):
            assert float((together[j][i] - ref[j]).abs().max()) <= tol, f"sequence {i}, step {j}: against plain"
            assert float((together[j][i] - alone[j][0]).abs().max()) <= 2 * tol, f"sequence {i}, step {j}: against alone"
    cfgb, _ = CONFIGS["B"]
    prompts = random_prompts(cfgb["vocab_size"], lengths, seed=43)
    feeds = random_prompts(cfgb["vocab_size"], [5] * n, seed=44)
    outs = []
    for graphs in (True, False):
        eng = tb.load(folders["B"], dtype="bfloat16", max_tokens=128 * n, max_slots=n + 1)
        eng.use_graphs = graphs
        outs.append(_decode_batch(eng, prompts, feeds, 5))
        assert bool(eng._graphs) == graphs
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_wider_than_the_graph_limit_runs_eagerly(dtype, folders):
    cfg, _ = CONFIGS["A"]
    prompts = random_prompts(cfg["vocab_size"], [3, 9, 1, 20, 5, 7], seed=51)
    feeds = random_prompts(cfg["vocab_size"], [4] * 6, seed=52)
    outs = []
    for limit in (4, 256, 0):
        eng = tb.load(folders["A"], dtype=dtype, max_tokens=1024)
        eng.graph_max_batch = limit
        six = _decode_batch(eng, prompts, feeds, 4)
        four = _decode_batch(eng, prompts[:4], feeds[:4], 4)
        assert (6 in eng._graphs) == (limit >= 6) and (4 in eng._graphs) == (limit >= 4)
        outs.append(six + four)
    for a, b, c in zip(*outs):
        assert torch.equal(a, b) and torch.equal(a, c)
