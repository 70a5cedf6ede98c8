"""Trace replay through bin/trace_run against the plain implementation.

The same requests are replayed (1) each alone and whole, (2) each alone with the last 32 tokens
one by one, (3) in batches of unequal lengths whose shorter requests end earlier, one batch after
another in a cache that holds only one batch, so slots and pages are used again -- in float32 and
in bfloat16, for every tiny configuration.  Every position's logits are compared.
"""
import pytest

from plain import llama_moe_plain as P
from tiny import CONFIGS, TraceRun, check_request, make_folder, n_moe_layers, random_prompts

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 11, 17, 40, 65, 97, 128], "B": [1, 9, 30, 64, 70, 100, 200], "dense": [3, 33, 64, 129],
           "C": [300, 70, 1, 420]}


def _k(cfg):
    return cfg.get("num_experts_per_tok", 0)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {name: make_folder(tmp, name) for name in CONFIGS}


def _collect(run, step, cfg, entries, got, routes):
    """File the logits and routes of one step under each request."""
    V, k, nl = cfg["vocab_size"], _k(cfg), n_moe_layers(cfg)
    nt = sum(len(e["tokens"]) for e in entries)
    lg = run.logits(step, V) if any(e["want"] for e in entries) else None
    rt = run.routes(step, nt, k) if nl else None
    row = tok = 0
    for e in entries:
        rid, n = e["id"], len(e["tokens"])
        base = e["_pos"]
        for w in e["want"]:
            got.setdefault(rid, {})[base + w] = lg[row].clone()
            row += 1
        if rt is not None:
            for j in range(n):
                routes.setdefault(rid, {})[base + j] = rt[:, tok + j, :]
        tok += n


def _entry(rid, tokens, pos):
    return {"id": rid, "tokens": tokens, "want": list(range(len(tokens))), "_pos": pos}


def _send(run, step, entries, end=(), log=None):
    clean = [{k: v for k, v in e.items() if not k.startswith("_")} for e in entries]
    if log is not None:
        log.append((step, clean, list(end)))
    run.step(step, clean, end)


def _verify(cfg, tensors, reqs, got, routes, dtype, label):
    import numpy as np
    nl = n_moe_layers(cfg)
    for rid, tokens in reqs.items():
        assert sorted(got[rid]) == list(range(len(tokens))), f"{label} {rid}: positions missing"
        r = None
        if nl:
            r = np.stack([routes[rid][p] for p in range(len(tokens))], axis=1)   # [layers, tokens, k]
        check_request(cfg, tensors, tokens, got[rid], r, dtype, f"{label} request {rid} ({len(tokens)} tokens)")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_replay_three_ways(name, dtype, folders, tmp_path):
    cfg, _ = CONFIGS[name]
    _, tensors = P.read_folder(folders[name])
    prompts = random_prompts(cfg["vocab_size"], LENGTHS[name], seed=1)
    # the cache holds one batch of mode 3 and nothing more: later batches must reuse what ended
    half = (len(prompts) + 1) // 2
    batches = [list(range(0, half)), list(range(half, len(prompts)))]
    max_tokens = max(sum((len(prompts[i]) + 63) // 64 * 64 for i in b) for b in batches)
    run = TraceRun(folders[name], dtype, str(tmp_path / "out"), max_tokens)
    step = 0
    sent = []      # the steps of (2) and (3), to be replayed once more through the CUDA-graph path
    try:
        # (1) each request alone and whole
        got, routes, reqs = {}, {}, {}
        for i, p in enumerate(prompts):
            rid = f"w{i}"
            reqs[rid] = p
            e = [_entry(rid, p, 0)]
            _send(run, step, e, end=[rid])
            _collect(run, step, cfg, e, got, routes)
            step += 1
        _verify(cfg, tensors, reqs, got, routes, dtype, "whole")

        # (2) each alone, the last 32 tokens one by one
        got, routes, reqs = {}, {}, {}
        for i, p in enumerate(prompts):
            rid = f"d{i}"
            reqs[rid] = p
            cut = max(1, len(p) - 32)
            e = [_entry(rid, p[:cut], 0)]
            _send(run, step, e, end=[rid] if cut == len(p) else [], log=sent)
            _collect(run, step, cfg, e, got, routes)
            step += 1
            for j in range(cut, len(p)):
                e = [_entry(rid, [p[j]], j)]
                _send(run, step, e, end=[rid] if j == len(p) - 1 else [], log=sent)
                _collect(run, step, cfg, e, got, routes)
                step += 1
        _verify(cfg, tensors, reqs, got, routes, dtype, "last 32 one by one")

        # (3) batches of unequal lengths; request i of a batch decodes its last (3 + 4 i) tokens,
        #     so the shorter ones end earlier; batch after batch in the same small cache
        got, routes, reqs = {}, {}, {}
        for b in batches:
            ids = {i: f"b{i}" for i in b}
            ndec = {i: min(len(prompts[i]) - 1, 3 + 4 * n) for n, i in enumerate(b)}
            for i in b:
                reqs[ids[i]] = prompts[i]
            e = [_entry(ids[i], prompts[i][:len(prompts[i]) - ndec[i]], 0) for i in b]
            ended = [ids[i] for i in b if ndec[i] == 0]
            _send(run, step, e, end=ended, log=sent)
            _collect(run, step, cfg, e, got, routes)
            step += 1
            for s in range(max(ndec.values())):
                live = [i for i in b if s < ndec[i]]
                e = [_entry(ids[i], [prompts[i][len(prompts[i]) - ndec[i] + s]], len(prompts[i]) - ndec[i] + s)
                     for i in live]
                ended = [ids[i] for i in live if s == ndec[i] - 1]
                _send(run, step, e, end=ended, log=sent)
                _collect(run, step, cfg, e, got, routes)
                step += 1
        _verify(cfg, tensors, reqs, got, routes, dtype, "unequal batches")
    finally:
        run.close()
    # Recording the experts switches CUDA graphs off.  The same steps once more as generation runs them (decode
    # steps replay a graph from their second use of a batch size on): the logits must not differ by a bit.
    import numpy as np
    again = TraceRun(folders[name], dtype, str(tmp_path / "graphs"), max_tokens, record_routing=False)
    try:
        for n, entries, end in sent:
            again.step(n, entries, end)
    finally:
        again.close()
    for n, entries, _ in sent:
        a = np.fromfile(str(tmp_path / "out" / f"{n}.f32"), dtype="<f4")
        b = np.fromfile(str(tmp_path / "graphs" / f"{n}.f32"), dtype="<f4")
        assert a.shape == b.shape and np.array_equal(a, b), f"step {n}: the graph path gives other logits"


def test_replay_rejects_overflow(folders, tmp_path):
    """More live tokens than --max-tokens is an error, not a wrong result."""
    cfg, _ = CONFIGS["A"]
    run = TraceRun(folders["A"], "float32", str(tmp_path / "out"), 64, record_routing=False)
    run.step(0, [{"id": "a", "tokens": list(range(60)), "want": [59]}])
    with pytest.raises(AssertionError):
        run.step(1, [{"id": "b", "tokens": list(range(10)), "want": [9]}])
    run.proc.kill()
    run.proc.wait()
