"""Configurations drawn at random -- head sizes 16 to 256, one to eight query heads per key/value head, widths and
vocabularies that are no powers of two, dense and with 2 to 33 experts, both rotary pairings, tied and untied
heads -- each run as a request that is cut at a random place and then decoded token by token.

float32: against the plain implementation, to 1e-4 of the largest |logit| (at least 1e-4).
bfloat16: against the plain implementation ROUNDING WHERE THE ENGINE STORES (``store=``), which is two to ten times
closer to the bfloat16 path than the unrounded one and so shows faults that rounding noise would hide.  What is left
is noise that no two bfloat16 implementations share: a value on a rounding boundary falls one way here and the other
way there (one unit roundoff u = 2^-8 of that value), and the prompt kernels also round the attention probabilities.
It grows with the depth, so the bound is 2 u (layers + 1) of the largest |logit|: 2^-6 for one layer, the package's
rule for its tiny models; a wrong mask, page, position or expert is off by tenths of the largest logit.
"""
import random

import pytest
import torch

import transformer_b200 as tb
from plain import llama_moe_plain as P
from tiny import check_request, n_moe_layers

pytestmark = pytest.mark.gpu


def random_config(rng):
    dh = rng.choice([16, 32, 48, 64, 64, 128, 128, 80, 96, 256])
    nkvh = rng.choice([1, 2, 3, 4])
    nh = nkvh * rng.choice([1, 1, 2, 3, 4, 5, 8])
    moe = rng.random() < 0.75
    cfg = {"model_type": "llama", "num_hidden_layers": rng.randint(1, 3), "hidden_size": 8 * rng.randint(4, 40),
           "num_attention_heads": nh, "num_key_value_heads": nkvh, "head_dim": dh,
           "intermediate_size": 8 * rng.randint(2, 30), "max_position_embeddings": rng.choice([128, 200, 320]),
           "vocab_size": rng.randint(50, 700), "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-4]),
           "rope_theta": rng.choice([1e4, 5e5, 123.0]), "tie_word_embeddings": rng.random() < 0.4,
           "rope_pairing": rng.choice(["adjacent", "half"])}
    if moe:
        cfg["num_local_experts"] = rng.choice([2, 3, 4, 5, 8, 16, 33])
        cfg["num_experts_per_tok"] = rng.randint(1, min(cfg["num_local_experts"], 6))
    return cfg


def _as_bfloat16(x):
    return x.bfloat16().float()


@pytest.mark.parametrize("seed", range(12))
def test_a_random_configuration(seed, tmp_path):
    rng = random.Random(1000 + seed)
    cfg = random_config(rng)
    folder = tb.write_random_model(str(tmp_path / "m"), cfg, seed=seed, std=0.1)
    _, tensors = P.read_folder(folder)
    n = rng.randint(20, min(cfg["max_position_embeddings"] - 1, 120))
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
    cut = rng.randint(1, n)
    for dtype in ("float32", "bfloat16"):
        engine = tb.load(folder, dtype=dtype, max_tokens=512)
        engine.use_graphs = False
        chosen = []
        engine.recorder = lambda name, run, t: chosen.append(t.cpu()) if name == "moe.topk_idx" else None
        slot = engine.open()
        rows = [engine.step([slot], [tokens[:cut]], [list(range(cut))]).cpu()]
        rows += [engine.step([slot], [[t]]).cpu() for t in tokens[cut:]]
        engine.close(slot)
        got = dict(enumerate(torch.cat(rows)))
        routes = None
        L = n_moe_layers(cfg)
        if L:
            steps = [chosen[i:i + L] for i in range(0, len(chosen), L)]                 # per step: [layers] of [nt, k]
            routes = torch.stack([torch.cat([s[l] for s in steps]) for l in range(L)]).numpy()
        if dtype == "float32":
            check_request(cfg, tensors, tokens, got, routes, dtype, f"{cfg}",
                          logit_tol=lambda biggest: 1e-4 * max(1.0, biggest))
        else:
            depth = cfg["num_hidden_layers"]
            check_request(cfg, tensors, tokens, got, routes, dtype, f"{cfg}", store=_as_bfloat16,
                          logit_tol=lambda biggest: 2 * 2.0 ** -8 * (depth + 1) * biggest)
        engine.cache.table.check()
