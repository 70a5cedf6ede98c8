"""The plain implementation checked against itself: independent restatements and invariances.

No output of the reference anchors it (the reference cannot be built here), so each part is
restated another way and the whole is checked for properties any right implementation has.
"""
import math

import pytest
import torch

from plain import llama_moe_plain as P
from tiny import CONFIGS, make_folder, random_prompts


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("plain")
    return {n: P.read_folder(make_folder(tmp, n), torch.float64) for n in CONFIGS}


def test_rms_norm_rowwise():
    x = torch.randn(3, 10, dtype=torch.float64)
    w = torch.randn(10, dtype=torch.float64)
    y = P.rms_norm(x, w, 1e-5)
    for r in range(3):
        ms = sum(float(v) ** 2 for v in x[r]) / 10
        for c in range(10):
            assert abs(float(y[r, c]) - float(x[r, c]) / math.sqrt(ms + 1e-5) * float(w[c])) < 1e-12


@pytest.mark.parametrize("pairing", ["adjacent", "half"])
def test_rope_is_a_rotation_and_relative(pairing):
    q = torch.randn(1, 1, 8, dtype=torch.float64)
    k = torch.randn(1, 1, 8, dtype=torch.float64)
    assert torch.allclose(P.rope(q, [0], 1e4, pairing), q)
    assert abs(float(P.rope(q, [5], 1e4, pairing).norm() - q.norm())) < 1e-12
    # scores depend on the distance only
    s1 = (P.rope(q, [7], 1e4, pairing) * P.rope(k, [3], 1e4, pairing)).sum()
    s2 = (P.rope(q, [104], 1e4, pairing) * P.rope(k, [100], 1e4, pairing)).sum()
    assert abs(float(s1 - s2)) < 1e-9


def test_attention_against_masked_matrix_form():
    n, nh, nkvh, dh = 7, 4, 2, 8
    q, k, v = (torch.randn(n, h, dh, dtype=torch.float64) for h in (nh, nkvh, nkvh))
    out = P.causal_attention(q, k, v)
    kk, vv = k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1)
    s = torch.einsum("ahd,bhd->hab", q, kk) / math.sqrt(dh)
    s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
    ref = torch.einsum("hab,bhd->ahd", torch.softmax(s, -1), vv)
    assert torch.allclose(out, ref, atol=1e-12)


def test_route_matches_full_softmax_renormalised():
    lg = torch.tensor([0.3, 2.0, -1.0, 2.0, 0.5], dtype=torch.float64)
    experts, w = P.route(lg, 3)
    assert experts == [1, 3, 4], "equal logits: the lower expert first"
    full = torch.softmax(lg, 0)
    assert torch.allclose(w, full[experts] / full[experts].sum())


def test_prefix_independence(models):
    """Causality: the logits of a prefix do not change when tokens follow."""
    for name, (cfg, t) in models.items():
        p = random_prompts(cfg["vocab_size"], [24], 3)[0]
        whole = P.forward(cfg, t, p)
        part = P.forward(cfg, t, p[:10])
        assert torch.allclose(whole[:10], part, atol=1e-10), name


def test_expert_permutation_invariance(models):
    cfg, t = models["A"]
    perm = [2, 0, 3, 1]
    t2 = dict(t)
    for i in range(cfg["num_hidden_layers"]):
        for n in ("ffn_gate_inp", "ffn_gate_up_exps", "ffn_down_exps"):
            t2[f"blk.{i}.{n}.weight"] = t[f"blk.{i}.{n}.weight"][perm]
    p = random_prompts(cfg["vocab_size"], [12], 4)[0]
    assert torch.allclose(P.forward(cfg, t, p), P.forward(cfg, t2, p), atol=1e-10)


def test_tied_equals_copied_head(models):
    cfg, t = models["B"]
    t2 = dict(t)
    t2["output.weight"] = t["token_embd.weight"].clone()
    p = random_prompts(cfg["vocab_size"], [9], 5)[0]
    assert torch.equal(P.forward(cfg, t, p), P.forward(cfg, t2, p))


def test_gqa_equals_repeated_heads(models):
    cfg, t = models["A"]
    nh, nkvh, dh, d = 4, 2, 16, 64
    cfg2 = dict(cfg, num_key_value_heads=nh)
    t2 = dict(t)
    for i in range(cfg["num_hidden_layers"]):
        w = t[f"blk.{i}.attn_qkv.weight"]
        q, k, v = w[:nh * dh], w[nh * dh:(nh + nkvh) * dh], w[(nh + nkvh) * dh:]
        rep = lambda m: m.reshape(nkvh, dh, d).repeat_interleave(nh // nkvh, dim=0).reshape(nh * dh, d)
        t2[f"blk.{i}.attn_qkv.weight"] = torch.cat([q, rep(k), rep(v)])
    p = random_prompts(cfg["vocab_size"], [10], 6)[0]
    assert torch.allclose(P.forward(cfg, t, p), P.forward(cfg2, t2, p), atol=1e-10)


def test_float32_close_to_float64(models, tmp_path):
    cfg, t64 = models["B"]
    t32 = {k: v.float() for k, v in t64.items()}
    p = random_prompts(cfg["vocab_size"], [20], 7)[0]
    a, b = P.forward(cfg, t64, p), P.forward(cfg, t32, p).double()
    assert float((a - b).abs().max()) < 2e-5


def test_sample_distribution():
    lg = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0])
    assert P.sample_distribution(lg, 0.0, 0, 1.0) == ([1], [1.0])
    ids, pr = P.sample_distribution(lg, 1.0, 2, 1.0)
    assert ids == [1, 3] and abs(pr[0] - 0.5) < 1e-12
    ids, pr = P.sample_distribution(lg, 0.5, 0, 0.6)
    assert ids == [1, 3] and abs(sum(pr) - 1) < 1e-12     # 2 x 0.4647 reaches 0.6, one alone does not
    ids, pr = P.sample_distribution(lg, 1.0, 0, 1.0)
    assert ids == [0, 1, 2, 3, 4]
