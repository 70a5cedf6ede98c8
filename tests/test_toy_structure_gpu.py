"""Toy structure of every kind the registries take beyond parts of a layer -- all defined HERE, registered, built
and stepped without a change to the library's files:

  * a cache kind "window" (a ring of the last W keys and values per slot, no pages) with a windowed attention
    mixer that uses it;
  * a block arrangement "parallel":  x += mixer(norm(x)) + feed_forward(norm(x))  with one norm;
  * a position encoding that is no rotation: a learned offset per position added to queries and keys (it has a
    parameter of its own, which travels with its mixer);
  * an embedding that adds learned absolute positions to the token rows;
  * a head that caps its logits:  cap * tanh(logits / cap).

The model made of them is held against a plain restatement in this file (whole sequences, float64).
"""
import dataclasses
import math
import os
from types import SimpleNamespace

import pytest
import torch
from safetensors.torch import load_file

import transformer_b200 as tb
from transformer_b200.architectures.generic import plan_from_spec
from transformer_b200.cache import CACHE_KINDS, CacheError, CacheStorage
from transformer_b200.config.registry import Architecture, register_architecture, unregister_architecture
from transformer_b200.parts import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, CacheNeed,
                                    Embedding, Head, LayerSpec, Mixer, ModelSpec, ParamDecl, PartSpec, Position, RunEntry)
from transformer_b200.parts.block import add_pending

pytestmark = pytest.mark.gpu


# ---- a cache kind and the mixer that uses it ---------------------------------------------------------------
class WindowStorage(CacheStorage):
    def __init__(self, need, runs, *, n_pages, max_slots, max_context, dtype, device):
        super().__init__(need, runs, n_pages=n_pages, max_slots=max_slots, max_context=max_context, dtype=dtype,
                         device=device)
        self.window = int(need.get()["window"])
        shape = (len(runs), max_slots, need.nkvh, self.window, need.dh)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.opened = []

    def view(self, index, writable):
        return SimpleNamespace(k=self.k[index], v=self.v[index], window=self.window, writable=writable)

    def open(self, slot):
        self.opened.append(slot)
        self.k[:, slot].fill_(float("nan"))      # whatever an earlier tenant left must never be read
        self.v[:, slot].fill_(float("nan"))

    @property
    def nbytes(self):
        return 2 * self.k.numel() * self.k.element_size()


class WindowAttention(Mixer):
    """Each token sees itself and the window - 1 tokens before it; no position encoding."""

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d, self.nh, self.dh, self.window = (int(params[k]) for k in ("width", "nh", "dh", "window"))

    def parameters(self):
        return {"wqkv": ParamDecl((3 * self.nh * self.dh, self.d)), "wo": ParamDecl((self.d, self.nh * self.dh))}

    def cache_need(self):
        return CacheNeed("window", self.nh, self.dh, (("window", self.window),))

    def forward(self, ctx, x1, out, cache, state):
        W, nh, dh = cache.window, self.nh, self.dh
        qkv = (x1.float() @ self.weights["wqkv"].float().T).view(-1, 3, nh, dh)
        o = torch.empty((x1.shape[0], nh, dh), dtype=torch.float32, device=x1.device)
        i = 0
        for b, n in enumerate(ctx.h_lens):
            slot = ctx.h_slots[b]
            for p in range(ctx.h_pos0[b], ctx.h_pos0[b] + n):
                cache.k[slot, :, p % W] = qkv[i, 1].to(cache.k.dtype)
                cache.v[slot, :, p % W] = qkv[i, 2].to(cache.v.dtype)
                ring = [q % W for q in range(max(0, p - W + 1), p + 1)]
                k, v = cache.k[slot][:, ring].float(), cache.v[slot][:, ring].float()      # [nh, seen, dh]
                s = torch.einsum("hd,hkd->hk", qkv[i, 0], k) / math.sqrt(dh)
                o[i] = torch.einsum("hk,hkd->hd", torch.softmax(s, -1), v)
                i += 1
        out.copy_((o.view(-1, nh * dh) @ self.weights["wo"].float().T).to(out.dtype))


# ---- an arrangement ----------------------------------------------------------------------------------------
class ParallelBlock:
    def __init__(self, spec, dtype, device):
        self.norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device)

    graph_safe = False

    def parts(self):
        return {"norm": self.norm, "mixer": self.mixer, "feed_forward": self.feed_forward}

    def forward(self, ctx, x, pending, cache_view, state):
        nt, d = x.shape
        x1 = ctx.scratch("parallel.x1", (nt, d), ctx.dtype)
        a = ctx.scratch("parallel.a", (nt, d), ctx.dtype)
        f = ctx.scratch("parallel.f", (nt, d), ctx.dtype)
        if not isinstance(pending, torch.Tensor):
            add_pending(ctx, x, pending)             # weighted rows of the block before: summed and added now
            pending = None
        self.norm.forward(ctx, x, pending, None, x1)
        self.mixer.forward(ctx, x1, a, cache_view, state)
        lazy = self.feed_forward.forward(ctx, x1, f)
        assert lazy is None
        x.add_(a.float())
        return f                                      # the next norm adds it


# ---- a position encoding that is no rotation, an embedding with positions, a capped head -----------------------
class LearnedOffsets(Position):
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.dh, self.positions = int(params["dh"]), int(params["positions"])

    def parameters(self):
        return {"offsets": ParamDecl((self.positions, self.dh))}

    def apply(self, ctx, qkv, nh, nkvh, dh):
        off = self.weights["offsets"][ctx.tok_pos.long()]                     # [nt, dh]
        qk = qkv[:, :(nh + nkvh) * dh].view(-1, nh + nkvh, dh)
        qk.copy_((qk.float() + off.float()[:, None, :]).to(qkv.dtype))


class LookupWithPositions(Embedding):
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.vocab, self.width, self.positions = (int(params[k]) for k in ("vocab", "width", "positions"))

    def parameters(self):
        return {"table": ParamDecl((self.vocab, self.width)), "where": ParamDecl((self.positions, self.width))}

    def forward(self, ctx, x):
        x.copy_(self.weights["table"][ctx.tok_ids.long()].float() + self.weights["where"][ctx.tok_pos.long()].float())


class CappedHead(Head):
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.vocab, self.width, self.cap = int(params["vocab"]), int(params["width"]), float(params["cap"])

    def parameters(self):
        return {"weight": ParamDecl((self.vocab, self.width))}

    def forward(self, ctx, xn, logits):
        logits.copy_(self.cap * torch.tanh(xn.float() @ self.weights["weight"].float().T / self.cap))


# ---- the model -----------------------------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class ToyConfig:
    width: int
    vocab: int
    context: int
    window: int
    cap: float
    model_type: str = "toy_structure"

    @classmethod
    def from_dict(cls, c):
        return cls(c["width"], c["vocab"], c["context"], c["window"], c["cap"])

    def to_dict(self):
        return dataclasses.asdict(self)


NH, NKVH, DH, DI = 3, 1, 16, 40


def toy_spec(c: ToyConfig) -> ModelSpec:
    rms = PartSpec.of("rmsnorm", width=c.width, eps=1e-5)
    learned = PartSpec.of("learned_offsets", dh=DH, positions=c.context)
    ff = PartSpec.of("swiglu", width=c.width, di=DI)
    first = LayerSpec(PartSpec.of("attention", width=c.width, nh=NH, nkvh=NKVH, dh=DH, position=learned), ff,
                      mixer_norm=rms, arrangement="parallel")
    second = LayerSpec(PartSpec.of("window_attention", width=c.width, nh=2, dh=DH, window=c.window), ff, rms, rms)
    return ModelSpec(width=c.width, vocab=c.vocab, max_context=c.context, layers=(first, second),
                     order=(RunEntry(0), RunEntry(1), RunEntry(1)),      # the windowed layer runs twice: two rings
                     embedding=PartSpec.of("lookup_with_positions", vocab=c.vocab, width=c.width, positions=c.context),
                     final_norm=rms, head=PartSpec.of("capped_linear", vocab=c.vocab, width=c.width, cap=c.cap))


@pytest.fixture()
def toys():
    CACHE_KINDS.register("window", WindowStorage)
    MIXERS.register("window_attention", WindowAttention)
    ARRANGEMENTS.register("parallel", ParallelBlock)
    POSITIONS.register("learned_offsets", LearnedOffsets)
    EMBEDDINGS.register("lookup_with_positions", LookupWithPositions)
    HEADS.register("capped_linear", CappedHead)
    register_architecture(Architecture("toy_structure", ToyConfig, toy_spec, lambda c: plan_from_spec(toy_spec(c))))
    yield
    unregister_architecture("toy_structure")
    for reg, kind in ((HEADS, "capped_linear"), (EMBEDDINGS, "lookup_with_positions"), (POSITIONS, "learned_offsets"),
                      (ARRANGEMENTS, "parallel"), (MIXERS, "window_attention"), (CACHE_KINDS, "window")):
        reg.unregister(kind)


CFG = {"model_type": "toy_structure", "width": 48, "vocab": 70, "context": 96, "window": 8, "cap": 0.5}


# ---- the model once more, plainly ----------------------------------------------------------------------------
def plain(folder, tokens, cfg=CFG):
    t = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    n = len(tokens)
    pos = torch.arange(n)

    def rms(x, w):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w

    def swiglu(x, p):
        gu = x @ t[p + ".wgu"].T
        return (gu[:, :DI] / (1 + torch.exp(-gu[:, :DI])) * gu[:, DI:]) @ t[p + ".wd"].T

    def attend(q, k, v, window):
        nh = q.shape[1]
        k, v = k.repeat_interleave(nh // k.shape[1], 1), v.repeat_interleave(nh // v.shape[1], 1)
        s = torch.einsum("ahd,bhd->hab", q, k) / math.sqrt(DH)
        seen = (pos[None, :] <= pos[:, None]) & (pos[None, :] > pos[:, None] - window)
        s = s.masked_fill(~seen, float("-inf"))
        return torch.einsum("hab,bhd->ahd", torch.softmax(s, -1), v).reshape(n, -1)

    x = t["embedding.table"][tokens] + t["embedding.where"][pos]
    # the parallel block with learned offsets on queries and keys
    x1 = rms(x, t["layers.0.norm.weight"])
    qkv = (x1 @ t["layers.0.mixer.wqkv"].T).view(n, NH + 2 * NKVH, DH)
    off = t["layers.0.mixer.position.offsets"][pos][:, None, :]
    a = attend(qkv[:, :NH] + off, qkv[:, NH:NH + NKVH] + off, qkv[:, NH + NKVH:], n) @ t["layers.0.mixer.wo"].T
    x = x + a + swiglu(x1, "layers.0.feed_forward")
    # the windowed layer, twice
    for _ in range(2):
        x1 = rms(x, t["layers.1.mixer_norm.weight"])
        qkv = (x1 @ t["layers.1.mixer.wqkv"].T).view(n, 3, 2, DH)
        x = x + attend(qkv[:, 0], qkv[:, 1], qkv[:, 2], cfg["window"]) @ t["layers.1.mixer.wo"].T
        x = x + swiglu(rms(x, t["layers.1.feed_forward_norm.weight"]), "layers.1.feed_forward")
    raw = rms(x, t["final_norm.weight"]) @ t["head.weight"].T
    plain.largest_uncapped = float(raw.abs().max())
    return cfg["cap"] * torch.tanh(raw / cfg["cap"])


def _whole(engine, tokens):
    s = engine.open()
    out = engine.step([s], [tokens], [list(range(len(tokens)))]).cpu()
    engine.close(s)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_toy_model_is_built_stepped_and_right(toys, dtype, tmp_path):
    folder = tb.write_random_model(str(tmp_path / "toy"), CFG, seed=9, std=0.12, dtype=dtype)
    engine = tb.load(folder, dtype=dtype, max_tokens=512, max_slots=2)
    assert [type(l).__name__ for l in engine.layers] == ["ParallelBlock", "Layer"]
    assert type(engine.embed).__name__ == "LookupWithPositions" and type(engine.head_part).__name__ == "CappedHead"
    kinds = sorted(g.need.kind for g in engine.cache.groups)
    assert kinds == ["full", "window"] and [len(g.runs) for g in engine.cache.groups if g.need.kind == "window"] == [2]
    assert not engine.graph_safe, "the toy block and the toy mixer run Python per step"
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, 70, (30,), generator=g).tolist()        # well past the window of 8
    b = torch.randint(0, 70, (11,), generator=g).tolist()
    ref_a, ref_b = plain(folder, a).float(), plain(folder, b).float()
    # the cap's slope is at most one, so the rounding rule of bfloat16 applies to the logits before the cap
    tol = 2e-4 if dtype == "float32" else 2.0 ** -6 * plain.largest_uncapped
    assert float((_whole(engine, a) - ref_a).abs().max()) <= tol
    assert float((_whole(engine, b) - ref_b).abs().max()) <= tol, "the slot's ring was used by another sequence before"
    # together: prompts of 12 and 4, then one token each; the shorter one ends earlier; then again in the other slots
    for _ in range(2):
        sa, sb = engine.open(), engine.open()
        lg = engine.step([sa, sb], [a[:12], b[:4]], [list(range(12)), list(range(4))]).cpu()
        got_a, got_b = [lg[:12]], [lg[12:]]
        for j in range(18):
            live = [(sa, a[12 + j], got_a)] + ([(sb, b[4 + j], got_b)] if 4 + j < len(b) else [])
            lg = engine.step([x[0] for x in live], [[x[1]] for x in live]).cpu()
            for i, x in enumerate(live):
                x[2].append(lg[i:i + 1])
            if 4 + j == len(b) - 1:
                engine.close(sb)
        engine.close(sa)
        assert float((torch.cat(got_a) - ref_a).abs().max()) <= tol
        assert float((torch.cat(got_b) - ref_b).abs().max()) <= tol
    assert float(ref_a.abs().max()) <= 0.5 and float(ref_a.abs().max()) > 0.3, "the cap is felt"
    window = [g for g in engine.cache.groups if g.need.kind == "window"][0]
    assert len(window.opened) == 6, "the storage class hears of every sequence that starts"
    out = tb.generate(engine, [a[:4], b[:7]], max_steps=5, stop_tokens=()).tokens
    assert [len(t) for t in out] == [5, 5]
    engine.cache.table.check()


def test_each_toy_changes_the_result(toys, tmp_path):
    """Window, offsets, positions in the embedding and the cap are really used: changing each changes the logits."""
    toks = list(range(3, 33))
    base = tb.write_random_model(str(tmp_path / "base"), CFG, seed=9, std=0.12, dtype="float32")
    ref = _whole(tb.load(base, dtype="float32", max_tokens=128), toks)
    wide = tb.write_random_model(str(tmp_path / "wide"), dict(CFG, window=64), seed=9, std=0.12, dtype="float32")
    out = _whole(tb.load(wide, dtype="float32", max_tokens=128), toks)
    assert torch.equal(out[:8], ref[:8]) and float((out[8:] - ref[8:]).abs().max()) > 1e-3, "the window cuts from token 9 on"
    capped = tb.write_random_model(str(tmp_path / "cap"), dict(CFG, cap=30.0), seed=9, std=0.12, dtype="float32")
    assert float(_whole(tb.load(capped, dtype="float32", max_tokens=128), toks).abs().max()) > 0.6
    eng = tb.load(base, dtype="float32", max_tokens=128)
    eng.layers[0].mixer.position.weights["offsets"].zero_()
    assert float((_whole(eng, toks) - ref).abs().max()) > 1e-3
    eng = tb.load(base, dtype="float32", max_tokens=128)
    eng.embed.weights["where"].zero_()
    assert float((_whole(eng, toks) - ref).abs().max()) > 1e-3


def test_an_unknown_kind_is_refused_by_name(toys, tmp_path):
    folder = tb.write_random_model(str(tmp_path / "toy"), CFG, seed=9, std=0.12)
    CACHE_KINDS.unregister("window")
    try:
        with pytest.raises(CacheError, match="unknown cache kind 'window'.*full"):
            tb.load(folder, dtype="float32", max_tokens=128)
    finally:
        CACHE_KINDS.register("window", WindowStorage)
    ARRANGEMENTS.unregister("parallel")
    try:
        with pytest.raises(ValueError, match="unknown block arrangement kind 'parallel'.*pre_norm"):
            tb.load(folder, dtype="float32", max_tokens=128)
    finally:
        ARRANGEMENTS.register("parallel", ParallelBlock)
