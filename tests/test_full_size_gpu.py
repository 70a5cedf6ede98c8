"""Layers of the benchmark's real sizes (one layer each, so the plain implementation stays fast):
the LLaMA-MoE-3.5B layer (width 4096, 32 heads of 128, 16 experts top-4 of width 688, vocabulary
32000) and a grouped-query layer in the manner of Mixtral (32 query heads on 8 key/value heads,
8 experts top-2).  Sizes like these reach code the tiny models do not: the vector kernels at width
4096, the decode products at real K and N with their tails, the tcgen05 products, heads of 128."""
import pytest
import torch

import transformer_b200 as tb
from plain import llama_moe_plain as P
from tiny import check_request, random_prompts

pytestmark = pytest.mark.gpu

LAYER_3_5B = {
    "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 128, "intermediate_size": 688, "num_local_experts": 16,
    "num_experts_per_tok": 4, "max_position_embeddings": 512, "vocab_size": 32000, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "tie_word_embeddings": True,
}
LAYER_GQA = {
    "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 1000, "num_local_experts": 8,
    "num_experts_per_tok": 2, "max_position_embeddings": 512, "vocab_size": 1000, "rms_norm_eps": 1e-5,
    "rope_theta": 1e6, "tie_word_embeddings": False,
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("full_size")
    out = {}
    for name, cfg in (("3.5b", LAYER_3_5B), ("gqa", LAYER_GQA)):
        folder = tb.write_random_model(str(tmp / name), cfg, seed=11, std=0.02)
        out[name] = (cfg, folder, P.read_folder(folder)[1])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["3.5b", "gqa"])
def test_one_real_layer_whole_then_token_by_token(name, dtype, models):
    cfg, folder, tensors = models[name]
    engine = tb.load(folder, dtype=dtype, max_tokens=1024)
    engine.use_graphs = False
    rec = []
    engine.recorder = lambda n, run, t: rec.append(t.cpu()) if n == "moe.topk_idx" else None
    prompts = random_prompts(cfg["vocab_size"], [140, 3, 70], seed=2)
    tail = 4                                           # the last tokens of each request go one by one, batched
    slots = [engine.open() for _ in prompts]
    got = [dict() for _ in prompts]
    routes = [dict() for _ in prompts]
    lg = engine.step(slots, [p[:-tail] if len(p) > tail else p[:1] for p in prompts],
                     [list(range(len(p) - tail)) if len(p) > tail else [0] for p in prompts]).cpu()
    r, row, tok = rec.pop(), 0, 0
    done = []
    for i, p in enumerate(prompts):
        n = len(p) - tail if len(p) > tail else 1
        for j in range(n):
            got[i][j] = lg[row + j]
            routes[i][j] = r[tok + j]
        row += n
        tok += n
        done.append(n)
    while any(d < len(p) for d, p in zip(done, prompts)):
        live = [i for i, p in enumerate(prompts) if done[i] < len(p)]
        lg = engine.step([slots[i] for i in live], [[prompts[i][done[i]]] for i in live]).cpu()
        r = rec.pop()
        for k, i in enumerate(live):
            got[i][done[i]] = lg[k]
            routes[i][done[i]] = r[k]
            done[i] += 1
    for i, p in enumerate(prompts):
        rt = torch.stack([routes[i][j] for j in range(len(p))])[None].numpy()      # [1 layer, tokens, k]
        check_request(cfg, tensors, p, got[i], rt, dtype, f"{name} request {i}")


def test_real_layer_through_cuda_graphs(models):
    """The same decode steps through the graph path (no recorder): equal to the eager ones bit for bit."""
    cfg, folder, _ = models["3.5b"]
    prompts = random_prompts(cfg["vocab_size"], [30, 9], seed=3)
    outs = []
    for graphs in (False, True):
        eng = tb.load(folder, dtype="bfloat16", max_tokens=512)
        eng.use_graphs = graphs
        slots = [eng.open() for _ in prompts]
        eng.step(slots, prompts)
        outs.append([eng.step(slots, [[5 + j], [7 + j]]).cpu().clone() for j in range(5)])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


LONG = {
    "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 1024, "max_position_embeddings": 16384,
    "vocab_size": 1000, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_pieces_then_decoding(dtype):
    """One real-size layer (grouped-query attention, dense feed-forward: no routing to tip) over 9,000 tokens: the
    prompt exceeds the 8,192 tokens a step takes at once, so it runs as two pieces, the second attending over what the
    first left in 128 pages of the cache; then three tokens one by one.  Logits at the first, a middle, the last position
    of each piece and at every decoded token against the plain implementation (float64 on the GPU, the same weights
    by the counter-based rule)."""
    from plain import counter_weights as C
    from plain import llama_moe_vectorized as PV
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    engine = tb.random_model(LONG, seed=21, dtype=dtype, std=0.02, max_tokens=9216, max_slots=1)
    tensors = {n: v.double() for n, v in C.llama_tensors(LONG, 21, 0.02, engine.device, tdt).items()}
    tokens = random_prompts(LONG["vocab_size"], [9003], seed=6)[0]
    want = [0, 4095, 8191, 8192, 8600, 8999]
    s = engine.open()
    got = [engine.step([s], [tokens[:9000]], [want]).cpu()]
    for t in tokens[9000:]:
        got.append(engine.step([s], [[t]]).cpu())
    engine.check_kernels()
    engine.close(s)
    got = torch.cat(got)
    store = None if dtype == "float32" else (lambda x: x.bfloat16().to(x.dtype))
    ref = PV.forward(LONG, tensors, tokens, want=want + [9000, 9001, 9002], store=store).float().cpu()
    tol = 1e-4 if dtype == "float32" else 2.0 ** -6 * float(ref.abs().max())
    worst = (got - ref).abs().max(dim=1).values
    assert float(worst.max()) <= tol, f"per position {worst.tolist()} against {tol}"
