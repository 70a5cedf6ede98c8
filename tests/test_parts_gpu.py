"""Each part of a layer alone (norm, position encoding, attention mixer, both feed-forwards, the
block arrangement) against the plain function of the same name, driven with a step context of its
own rather than through the model."""
import pytest
import torch

import transformer_b200 as tb
from plain import llama_moe_plain as P
from tiny import BF16_REL_TOL, CONFIGS, make_folder
from transformer_b200.engine.context import StepContext
from transformer_b200.parts import FEED_FORWARDS, MIXERS, NORMS, POSITIONS, PartSpec
from transformer_b200.parts.base import WeightedRows

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("part_models")
    return {n: make_folder(tmp, n) for n in CONFIGS}


def _ctx(engine, lens, pos0=None):
    """A step context for fresh sequences of the given lengths (pos0: tokens already in the cache)."""
    slots = [engine.open() for _ in lens]
    pos0 = pos0 or [0] * len(lens)
    for s, p, n in zip(slots, pos0, lens):
        engine.cache.extend(s, p + n)
    tokens = [[0] * n for n in lens]
    return StepContext(engine, slots, tokens, pos0, [], engine._tile_sizes), slots


def _close(engine, slots):
    for s in slots:
        engine.close(s)


def _tol(dtype, ref):
    return 2e-5 * max(1.0, float(ref.abs().max())) if dtype == "float32" else BF16_REL_TOL * float(ref.abs().max())


def test_registries_know_the_built_in_kinds():
    assert "rmsnorm" in NORMS.kinds() and "attention" in MIXERS.kinds() and "rope" in POSITIONS.kinds()
    assert {"moe", "swiglu"} <= set(FEED_FORWARDS.kinds())
    with pytest.raises(ValueError, match="unknown mixer kind"):
        MIXERS.build(PartSpec.of("no_such_mixer"), torch.float32, torch.device("cuda"))


@pytest.mark.parametrize("name", ["A", "B"])
def test_rope_table(name, folders):
    cfg, _ = CONFIGS[name]
    eng = tb.load(folders[name], dtype="float32", max_tokens=64)
    rope = eng.layers[0].mixer.position
    cos, sin = rope.tables()
    dh = cfg["head_dim"]
    assert cos.shape == (cfg["max_position_embeddings"], dh // 2)
    for p in (0, 1, 77, cfg["max_position_embeddings"] - 1):
        for i in (0, 1, dh // 2 - 1):
            ang = p * cfg["rope_theta"] ** (-2.0 * i / dh)
            assert abs(float(cos[p, i]) - __import__("math").cos(ang)) < 1e-6
            assert abs(float(sin[p, i]) - __import__("math").sin(ang)) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype, folders):
    eng = tb.load(folders["B"], dtype=dtype, max_tokens=256)
    d, eps = 96, CONFIGS["B"][0]["rms_norm_eps"]
    norm = eng.layers[1].feed_forward_norm
    ctx, slots = _ctx(eng, [9])
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, d, generator=g).cuda()
    delta = torch.randn(9, d, generator=g).to(eng.dtype).cuda()
    y = torch.empty(9, d, dtype=eng.dtype, device="cuda")
    x0 = x.clone()
    norm.forward(ctx, x, delta, None, y)
    v = x0.double() + delta.double()
    ref = P.rms_norm(v.cpu(), norm.weights["weight"].double().cpu(), eps)
    assert torch.allclose(x.double(), v, atol=1e-6)
    assert float((y.double().cpu() - ref).abs().max()) <= _tol(dtype, ref)
    # the un-summed output of the experts, summed inside the norm
    rows = torch.randn(18, d, generator=g).to(eng.dtype).cuda()
    index = torch.randperm(18, generator=g).to(torch.int32).cuda()
    w = torch.rand(9, 2, generator=g).cuda()
    x = x0.clone()
    norm.forward(ctx, x, WeightedRows(rows, index, w, 2), None, y)
    summed = (rows.double()[index.long()].reshape(9, 2, d) * w.double()[:, :, None]).sum(1)
    ref = P.rms_norm((x0.double() + summed).cpu(), norm.weights["weight"].double().cpu(), eps)
    assert float((y.double().cpu() - ref).abs().max()) <= _tol(dtype, ref)
    _close(eng, slots)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_attention_mixer_part(name, dtype, folders):
    cfg, _ = CONFIGS[name]
    _, t = P.read_folder(folders[name])
    eng = tb.load(folders[name], dtype=dtype, max_tokens=512)
    mixer = eng.layers[1].mixer
    lens = [70, 5, 1]
    ctx, slots = _ctx(eng, lens)
    g = torch.Generator().manual_seed(1)
    x1 = torch.randn(sum(lens), cfg["hidden_size"], generator=g).to(eng.dtype).cuda()
    out = torch.empty_like(x1)
    mixer.forward(ctx, x1, out, eng.cache.view(1), None)
    sz = P.sizes(cfg)
    lo = 0
    for n in lens:
        ref = P.attention_mixer(x1[lo:lo + n].float().cpu(), t["blk.1.attn_qkv.weight"], t["blk.1.attn_output.weight"],
                                list(range(n)), sz)
        assert float((out[lo:lo + n].float().cpu() - ref).abs().max()) <= _tol(dtype, ref), f"sequence of {n}"
        lo += n
    # one more token for each: the mixer reads what the first step left in the cache
    ctx2 = StepContext(eng, slots, [[0]] * 3, lens, [], eng._tile_sizes)
    for s in slots:
        eng.cache.extend(s, 1)
    x2 = torch.randn(3, cfg["hidden_size"], generator=g).to(eng.dtype).cuda()
    out2 = torch.empty_like(x2)
    ctx2 = StepContext(eng, slots, [[0]] * 3, lens, [], eng._tile_sizes)
    mixer.forward(ctx2, x2, out2, eng.cache.view(1), None)
    lo = 0
    for b, n in enumerate(lens):
        both = torch.cat([x1[lo:lo + n], x2[b:b + 1]]).float().cpu()
        ref = P.attention_mixer(both, t["blk.1.attn_qkv.weight"], t["blk.1.attn_output.weight"], list(range(n + 1)), sz)
        assert float((out2[b].float().cpu() - ref[-1]).abs().max()) <= _tol(dtype, ref), f"decode after {n}"
        lo += n
    _close(eng, slots)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,nt", [("A", 7), ("B", 40), ("C", 300)])
def test_moe_part(name, nt, dtype, folders):
    """Router, dispatch, expert products and the (deferred) weighted sum against the per-token loop;
    tokens whose k-th and (k+1)-th router logits nearly tie are left out of the comparison."""
    cfg, _ = CONFIGS[name]
    _, t = P.read_folder(folders[name])
    eng = tb.load(folders[name], dtype=dtype, max_tokens=512)
    ff = eng.layers[0].feed_forward
    ctx, slots = _ctx(eng, [nt])
    g = torch.Generator().manual_seed(2)
    x1 = torch.randn(nt, cfg["hidden_size"], generator=g).to(eng.dtype).cuda()
    out = torch.empty_like(x1)
    res = ff.forward(ctx, x1, out)
    assert isinstance(res, WeightedRows)
    from transformer_b200.parts.feed_forward import sum_weighted_rows
    sum_weighted_rows(res, out)
    margins = []
    ref = P.moe_feed_forward(x1.float().cpu(), t["blk.0.ffn_gate_inp.weight"], t["blk.0.ffn_gate_up_exps.weight"],
                             t["blk.0.ffn_down_exps.weight"], cfg["num_experts_per_tok"], margins=margins)
    clear = [a for a, (_, gap, big) in enumerate(margins) if gap > 2 * BF16_REL_TOL * big]
    assert len(clear) > nt * 0.8
    assert float((out.float().cpu()[clear] - ref[clear]).abs().max()) <= 2 * _tol(dtype, ref)
    _close(eng, slots)


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward_part(dtype, folders):
    cfg, _ = CONFIGS["dense"]
    _, t = P.read_folder(folders["dense"])
    eng = tb.load(folders["dense"], dtype=dtype, max_tokens=256)
    ff = eng.layers[1].feed_forward
    ctx, slots = _ctx(eng, [11])
    x1 = torch.randn(11, cfg["hidden_size"], generator=torch.Generator().manual_seed(3)).to(eng.dtype).cuda()
    out = torch.empty_like(x1)
    assert ff.forward(ctx, x1, out) is None
    ref = P.dense_feed_forward(x1.float().cpu(), t["blk.1.ffn_gate_up.weight"], t["blk.1.ffn_down.weight"])
    assert float((out.float().cpu() - ref).abs().max()) <= _tol(dtype, ref)
    _close(eng, slots)


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_arrangement(dtype, folders):
    """x += mixer(norm(x)); x += feed_forward(norm(x)) with the sums deferred into the next norm."""
    cfg, _ = CONFIGS["dense"]
    _, t = P.read_folder(folders["dense"])
    eng = tb.load(folders["dense"], dtype=dtype, max_tokens=256)
    n = 13
    ctx, slots = _ctx(eng, [n])
    x = torch.randn(n, cfg["hidden_size"], generator=torch.Generator().manual_seed(4)).cuda()
    x0 = x.clone()
    pending = eng.layers[0].forward(ctx, x, None, eng.cache.view(0), None)
    total = x.double().cpu() + pending.double().cpu()
    ref = P.block(x0.double().cpu(), {k: v.double() for k, v in t.items()}, 0, list(range(n)), P.sizes(cfg))
    assert float((total - ref).abs().max()) <= _tol(dtype, ref)
    _close(eng, slots)
