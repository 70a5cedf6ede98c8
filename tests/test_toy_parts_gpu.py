"""Toy parts of every other kind -- a feed-forward with routing, a norm that does not take the experts' weighted
rows, a position encoding -- defined HERE, registered, built and stepped without a change to the library's files.

  * "sign_gate" (feed-forward): each token goes through one of two square maps, chosen by the sign of a learned
    projection of the token;
  * "center_scale" (norm): y = (x - mean(x)) * w.  It sums a plain delta only, so the block must first add up the
    weighted rows that the mixture of experts before it left pending;
  * "rope_scaled" (position): rotary angles of position / scale; the attention mixer asks a position part for
    its ``rotation()`` (cos, sin, pairing) and knows nothing else about it.
"""
import dataclasses

import pytest
import torch

import transformer_b200 as tb
from transformer_b200.architectures.generic import plan_from_spec
from transformer_b200.config.registry import Architecture, register_architecture, unregister_architecture
from transformer_b200.parts import (FEED_FORWARDS, NORMS, POSITIONS, FeedForward, LayerSpec, ModelSpec, Norm, ParamDecl,
                                    PartSpec, RunEntry)
from transformer_b200.parts.base import Position

pytestmark = pytest.mark.gpu


class SignGate(FeedForward):
    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])

    def parameters(self):
        return {"gate": ParamDecl((1, self.d)), "a": ParamDecl((self.d, self.d)), "b": ParamDecl((self.d, self.d))}

    def forward(self, ctx, x1, out):
        x = x1.float()
        side = (x @ self.weights["gate"].float().T) > 0                       # [nt, 1]: the route of each token
        ya, yb = x @ self.weights["a"].float().T, x @ self.weights["b"].float().T
        out.copy_(torch.where(side, ya, yb).to(out.dtype))
        ctx.record("sign_gate.side", side)


class CenterScale(Norm):
    takes_weighted_rows = False

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])

    def parameters(self):
        return {"weight": ParamDecl((self.d,), "norm", "ones")}

    def forward(self, ctx, x, delta, rows, y):
        assert delta is None or isinstance(delta, torch.Tensor), "the block sums weighted rows for this norm"
        if rows is None:
            if delta is not None:
                x.add_(delta.float())                                          # the stream, in place, in float
            v = x
        else:
            v = x[rows.long()] + (delta[rows.long()].float() if delta is not None else 0.0)
        y.copy_(((v - v.mean(dim=1, keepdim=True)) * self.weights["weight"].float()).to(y.dtype))


class RopeScaled(Position):
    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.dh, self.theta = int(params["dh"]), float(params["theta"])
        self.scale, self.positions = float(params["scale"]), int(params["positions"])
        self._tables = None

    def rotation(self):
        if self._tables is None:
            i = torch.arange(self.dh // 2, dtype=torch.float64)
            ang = (torch.arange(self.positions, dtype=torch.float64) / self.scale)[:, None] * \
                torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.dh)[None, :]
            self._tables = (torch.cos(ang).float().contiguous().to(self.device),
                            torch.sin(ang).float().contiguous().to(self.device))
        return self._tables + (0,)


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    width: int
    vocab: int
    context: int
    scale: float
    model_type: str = "toy_parts"

    @classmethod
    def from_dict(cls, c):
        return cls(c["width"], c["vocab"], c["context"], c["scale"], c["model_type"])

    def to_dict(self):
        return dataclasses.asdict(self)


def toy_spec(c: ToyConfig) -> ModelSpec:
    rms = PartSpec.of("rmsnorm", width=c.width, eps=1e-5)
    center = PartSpec.of("center_scale", width=c.width)
    scaled = PartSpec.of("rope_scaled", dh=16, theta=10000.0, scale=c.scale, positions=c.context)
    rope = PartSpec.of("rope", dh=16, theta=10000.0, pairing="adjacent", positions=c.context)
    first = LayerSpec(PartSpec.of("attention", width=c.width, nh=3, nkvh=1, dh=16, position=scaled),
                      PartSpec.of("moe", width=c.width, di=24, nexp=4, nexp_use=2), rms, rms)
    # this layer's first norm meets the weighted rows the experts above left pending, and cannot take them
    second = LayerSpec(PartSpec.of("attention", width=c.width, nh=3, nkvh=3, dh=16, position=rope),
                       PartSpec.of("sign_gate", width=c.width), center, rms)
    return ModelSpec(width=c.width, vocab=c.vocab, max_context=c.context, layers=(first, second),
                     order=(RunEntry(0), RunEntry(1)), embedding=PartSpec.of("lookup", vocab=c.vocab, width=c.width),
                     final_norm=center, head=PartSpec.of("linear", vocab=c.vocab, width=c.width, tied=False))


@pytest.fixture()
def toys_registered():
    FEED_FORWARDS.register("sign_gate", SignGate)
    NORMS.register("center_scale", CenterScale)
    POSITIONS.register("rope_scaled", RopeScaled)
    register_architecture(Architecture("toy_parts", ToyConfig, toy_spec, lambda c: plan_from_spec(toy_spec(c))))
    yield
    unregister_architecture("toy_parts")
    POSITIONS.unregister("rope_scaled")
    NORMS.unregister("center_scale")
    FEED_FORWARDS.unregister("sign_gate")


CFG = {"model_type": "toy_parts", "width": 48, "vocab": 60, "context": 128, "scale": 4.0}


def _logits(engine, tokens):
    s = engine.open()
    out = engine.step([s], [tokens], [list(range(len(tokens)))]).cpu()
    engine.close(s)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_parts_are_registered_built_and_stepped(toys_registered, dtype, tmp_path):
    folder = tb.write_random_model(str(tmp_path / "toy"), CFG, seed=5, std=0.2)
    engine = tb.load(folder, dtype=dtype, max_tokens=512)
    kinds = [(type(l.mixer_norm).__name__, type(l.mixer.position).__name__, type(l.feed_forward).__name__)
             for l in engine.layers]
    assert kinds == [("RMSNorm", "RopeScaled", "MoE"), ("CenterScale", "Rope", "SignGate")]
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, 60, (70,), generator=g).tolist()      # crosses a page of the cache
    b = torch.randint(0, 60, (11,), generator=g).tolist()
    sides = []
    engine.recorder = lambda name, run, t: sides.append(t.cpu()) if name == "sign_gate.side" else None
    engine.use_graphs = False
    whole_a, whole_b = _logits(engine, a), _logits(engine, b)
    assert 0 < int(torch.cat(sides).sum()) < len(a) + len(b), "both routes of the toy feed-forward are taken"
    engine.recorder = None
    engine.use_graphs = True
    # together, in pieces, then one token each; the shorter one ends earlier
    sa, sb = engine.open(), engine.open()
    got_a, got_b = [], []
    lg = engine.step([sa, sb], [a[:50], b[:6]], [list(range(50)), list(range(6))]).cpu()
    got_a.append(lg[:50])
    got_b.append(lg[50:])
    for j in range(20):
        live = [(sa, a[50 + j], got_a)] + ([(sb, b[6 + j], got_b)] if 6 + j < len(b) else [])
        lg = engine.step([x[0] for x in live], [[x[1]] for x in live]).cpu()
        for i, x in enumerate(live):
            x[2].append(lg[i:i + 1])
        if 6 + j == len(b) - 1:
            engine.close(sb)
    engine.close(sa)
    tol = 2e-4 if dtype == "float32" else 2 * 2.0 ** -6 * float(whole_a.abs().max())
    assert float((torch.cat(got_a) - whole_a).abs().max()) <= tol
    assert float((torch.cat(got_b) - whole_b).abs().max()) <= tol
    out = tb.generate(engine, [a[:4], b[:7]], max_steps=5, stop_tokens=()).tokens
    assert [len(t) for t in out] == [5, 5]
    engine.cache.table.check()


def test_the_toy_position_is_what_the_attention_uses(toys_registered, tmp_path):
    """With a scale of 1 the toy encoding is the built-in one: the same logits to the bit; with 4 they differ from
    the second token on (the first has position 0 either way)."""
    toks = [3, 14, 15, 9, 26, 5, 35, 8]
    outs = {}
    for scale in (1.0, 4.0):
        f = tb.write_random_model(str(tmp_path / f"s{scale}"), dict(CFG, scale=scale), seed=5, std=0.2)
        outs[scale] = _logits(tb.load(f, dtype="float32", max_tokens=128), toks)

    def builtin_spec(c):
        s = toy_spec(c)
        att = s.layers[0].mixer
        plain = PartSpec.of("attention", **{**att.get(), "position": PartSpec.of(
            "rope", dh=16, theta=10000.0, pairing="adjacent", positions=c.context)})
        return dataclasses.replace(s, layers=(dataclasses.replace(s.layers[0], mixer=plain), s.layers[1]))
    register_architecture(Architecture("toy_parts_builtin_rope", ToyConfig, builtin_spec,
                                       lambda c: plan_from_spec(builtin_spec(c))))
    try:
        f = tb.write_random_model(str(tmp_path / "builtin"), dict(CFG, model_type="toy_parts_builtin_rope", scale=1.0),
                                  seed=5, std=0.2)
        ref = _logits(tb.load(f, dtype="float32", max_tokens=128), toks)
    finally:
        unregister_architecture("toy_parts_builtin_rope")
    assert torch.equal(outs[1.0], ref)
    assert torch.equal(outs[4.0][0], ref[0]) and float((outs[4.0][1:] - ref[1:]).abs().max()) > 1e-3
