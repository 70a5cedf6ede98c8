"""The vectorised plain implementation is the loop version, to rounding: every tiny configuration in float64,
free and forced routes, margins, the rounding hook; and the tests' restatement of the random-weight rule is the
package's, bit for bit."""
import numpy as np
import pytest
import torch

from plain import counter_weights as C
from plain import llama_moe_plain as P
from plain import llama_moe_vectorized as PV
from tiny import CONFIGS, make_folder, random_prompts


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("plain_v")
    return {n: P.read_folder(make_folder(tmp, n), torch.float64) for n in CONFIGS}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_vectorised_equals_the_loops(name, models):
    cfg, t = models[name]
    for n, seed in ((1, 3), (37, 4), (70, 5)):
        tokens = random_prompts(cfg["vocab_size"], [n], seed=seed)[0]
        m1, m2 = [], []
        a = P.forward(cfg, t, tokens, margins_out=m1)
        b = PV.forward(cfg, t, tokens, margins_out=m2)
        assert float((a - b).abs().max()) <= 1e-6 * max(1.0, float(a.abs().max()))
        for l1, l2 in zip(m1, m2):
            for (e1, g1, b1), (e2, g2, b2) in zip(l1, l2):
                assert e1 == e2 and abs(g1 - g2) < 1e-9 and abs(b1 - b2) < 1e-9
    want = [0, 5, 36]
    tokens = random_prompts(cfg["vocab_size"], [37], seed=4)[0]
    a, b = P.forward(cfg, t, tokens, want=want), PV.forward(cfg, t, tokens, want=want)
    assert a.shape[0] == 3 and float((a - b).abs().max()) <= 1e-6 * max(1.0, float(a.abs().max()))


@pytest.mark.parametrize("name", ["A", "B"])
def test_forced_routes_and_the_rounding_hook_agree_too(name, models):
    cfg, t = models[name]
    E, k, L = cfg["num_local_experts"], cfg["num_experts_per_tok"], cfg["num_hidden_layers"]
    tokens = random_prompts(cfg["vocab_size"], [23], seed=9)[0]
    g = torch.Generator().manual_seed(1)
    forced = [[torch.randperm(E, generator=g)[:k].tolist() for _ in tokens] for _ in range(L)]
    store = lambda x: x.bfloat16().to(x.dtype)
    a = P.forward(cfg, t, tokens, forced_routes=forced, store=store)
    b = PV.forward(cfg, t, tokens, forced_routes=forced, store=store)
    # with rounding to bfloat16 at every store, a last-bit difference before a store can become a bfloat16 step
    assert float((a - b).abs().max()) <= 2.0 ** -7 * float(a.abs().max())
    a = P.forward(cfg, t, tokens, forced_routes=forced)
    b = PV.forward(cfg, t, tokens, forced_routes=forced)
    assert float((a - b).abs().max()) <= 1e-6 * max(1.0, float(a.abs().max()))
    free = PV.forward(cfg, t, tokens)
    assert float((free - b).abs().max()) > 1e-3, "forcing other experts must change the result"


def test_layer_by_layer_tensors_give_the_same(models):
    cfg, t = models["B"]
    tokens = random_prompts(cfg["vocab_size"], [19], seed=2)[0]
    ends = {n: v for n, v in t.items() if not n.startswith("blk.")}
    walked = PV.forward(cfg, ends, tokens, tensors_of_layer=lambda i: {n: v for n, v in t.items()
                                                                       if n.startswith(f"blk.{i}.")})
    assert torch.equal(walked, PV.forward(cfg, t, tokens))


def test_the_weight_rule_restated_is_the_packages_rule():
    from transformer_b200.weights import counter_random as R
    for seed, name, shape, std, first in ((0, "token_embd.weight", (7, 33), 0.02, 0),
                                          (123456789, "blk.31.ffn_gate_up_exps.weight", (3, 10, 9), 0.1, 0),
                                          (2 ** 40 + 5, "x", (1001,), 1.0, 987654321)):
        n = int(np.prod(shape))
        mine = C.values(seed, name, shape, std, first=first)
        theirs = torch.from_numpy(R.normal_values(seed, name, first, n, std)).view(*shape)
        assert torch.equal(mine, theirs)
    v = C.values(1, "a", (1 << 18,), 0.02)
    assert abs(float(v.mean())) < 2e-4 and abs(float(v.std()) - 0.02) < 2e-4
    assert float(v.abs().max()) <= 0.02 * 4.9
    assert not torch.equal(v, C.values(2, "a", (1 << 18,), 0.02)) and not torch.equal(v, C.values(1, "b", (1 << 18,), 0.02))
    # a known value, so that the rule itself cannot drift unnoticed (computed by hand from the definition)
    base = R.stream_base(0, "w")
    h0, h1 = R.mix64_int(base), R.mix64_int((base + R.G) & R.MASK)
    c = sum((h >> (16 * f)) & 0xFFFF for h in (h0, h1) for f in range(4)) - 4 * 65535
    assert float(C.values(0, "w", (1,), 0.02)[0]) == float(np.float32(c) * np.float32(0.02 / R.SIGMA))


def test_a_written_folder_holds_the_rule(tmp_path):
    import transformer_b200 as tb
    cfg, seed = CONFIGS["B"]
    for dtype, tdt in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        folder = tb.write_random_model(str(tmp_path / dtype), cfg, seed=seed, dtype=dtype, std=0.05)
        _, read = P.read_folder(folder)
        mine = C.llama_tensors(cfg, seed, 0.05, dtype=tdt)
        assert sorted(read) == sorted(mine)
        for n in mine:
            assert torch.equal(read[n], mine[n]), n
