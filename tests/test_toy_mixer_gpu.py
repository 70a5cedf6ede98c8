"""A mixer with state of its own, a model that runs a layer twice and lets a run read another
run's cache -- all defined HERE, registered, built with random weights and stepped, without a
change to the library's files.

The toy mixer is a leaky running sum: for every sequence it keeps s (one vector of the model's
width, fixed size), and for each token  s <- decay * s + x1,  out = W s.  Its state lives in the
cache's per-sequence state tensor: zero when a sequence starts, carried from step to step.
"""
import dataclasses

import pytest
import torch

import transformer_b200 as tb
from transformer_b200.architectures.generic import plan_from_spec
from transformer_b200.config.registry import Architecture, register_architecture, unregister_architecture
from transformer_b200.parts import MIXERS, LayerSpec, Mixer, ModelSpec, ParamDecl, PartSpec, RunEntry, StateNeed

pytestmark = pytest.mark.gpu


class RunningSum(Mixer):
    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d, self.decay = int(params["width"]), float(params["decay"])

    def parameters(self):
        return {"w": ParamDecl((self.d, self.d))}

    def state_need(self):
        return StateNeed((self.d,), torch.float32)

    def forward(self, ctx, x1, out, cache, state):
        assert cache is None and state is not None
        w = self.weights["w"].float()
        lo = 0
        for b, n in enumerate(ctx.h_lens):            # plain torch: a toy needs no kernel of its own
            s = state[ctx.h_slots[b]]
            for i in range(lo, lo + n):
                s.mul_(self.decay).add_(x1[i].float())
                out[i] = (w @ s).to(out.dtype)
            lo += n


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    width: int
    vocab: int
    context: int
    decay: float

    @classmethod
    def from_dict(cls, c):
        return cls(c["width"], c["vocab"], c["context"], c["decay"])

    def to_dict(self):
        return {"model_type": "toy_running_sum", **dataclasses.asdict(self)}


def toy_spec(c: ToyConfig) -> ModelSpec:
    norm = PartSpec.of("rmsnorm", width=c.width, eps=1e-5)
    rope = PartSpec.of("rope", dh=16, theta=10000.0, pairing="adjacent", positions=c.context)
    toy = LayerSpec(PartSpec.of("running_sum", width=c.width, decay=c.decay), PartSpec.of("swiglu", width=c.width, di=24),
                    norm, norm)
    att = LayerSpec(PartSpec.of("attention", width=c.width, nh=2, nkvh=1, dh=16, position=rope),
                    PartSpec.of("moe", width=c.width, di=16, nexp=3, nexp_use=2), norm, norm)
    # layer 0 runs twice (two states), layer 1 runs twice and its second run reads the first run's cache
    order = (RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_of=1))
    return ModelSpec(width=c.width, vocab=c.vocab, max_context=c.context, layers=(toy, att), order=order,
                     embedding=PartSpec.of("lookup", vocab=c.vocab, width=c.width), final_norm=norm,
                     head=PartSpec.of("linear", vocab=c.vocab, width=c.width, tied=True))


@pytest.fixture()
def toy_registered():
    MIXERS.register("running_sum", RunningSum)
    arch = register_architecture(Architecture("toy_running_sum", ToyConfig, toy_spec,
                                              lambda c: plan_from_spec(toy_spec(c))))
    yield arch
    unregister_architecture("toy_running_sum")
    MIXERS.unregister("running_sum")


CFG = {"model_type": "toy_running_sum", "width": 40, "vocab": 50, "context": 96, "decay": 0.9}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_is_registered_built_and_stepped(toy_registered, dtype, tmp_path):
    folder = tb.write_random_model(str(tmp_path / "toy"), CFG, seed=3, std=0.2)
    engine = tb.load(folder, dtype=dtype, max_tokens=256)
    assert [type(l.mixer).__name__ for l in engine.layers] == ["RunningSum", "Attention"]
    assert sorted(engine.cache.state) == [0, 2], "a state tensor for each run of the toy layer"
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].k.shape[0] == 1, "one run owns a cache, one borrows it"
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, 50, (30,), generator=g).tolist()
    b = torch.randint(0, 50, (9,), generator=g).tolist()
    # whole, alone
    s = engine.open()
    whole_a = engine.step([s], [a], [list(range(len(a)))]).cpu()
    engine.close(s)
    s = engine.open()                                         # the same slot again: its state must be zero
    whole_b = engine.step([s], [b], [list(range(len(b)))]).cpu()
    engine.close(s)
    # together, in pieces: 20 + 5, then one token each; the shorter one ends earlier
    sa, sb = engine.open(), engine.open()
    got_a, got_b = [], []
    lg = engine.step([sa, sb], [a[:20], b[:5]], [list(range(20)), list(range(5))]).cpu()
    got_a.append(lg[:20])
    got_b.append(lg[20:])
    for j in range(10):
        live = [(sa, a[20 + j], got_a)] + ([(sb, b[5 + j], got_b)] if 5 + j < len(b) else [])
        lg = engine.step([x[0] for x in live], [[x[1]] for x in live]).cpu()
        for i, x in enumerate(live):
            x[2].append(lg[i:i + 1])
        if 5 + j == len(b) - 1:
            engine.close(sb)
    engine.close(sa)
    tol = 2e-4 if dtype == "float32" else 2.0 ** -6 * float(whole_a.abs().max())
    assert float((torch.cat(got_a) - whole_a).abs().max()) <= tol
    assert float((torch.cat(got_b) - whole_b).abs().max()) <= tol
    assert not torch.allclose(whole_a[5:9], whole_b[5:9], atol=1e-3), "the model does depend on its input"
    # generation works on it too
    out = tb.generate(engine, [a[:4], b[:7]], max_steps=5, stop_tokens=()).tokens
    assert [len(t) for t in out] == [5, 5]
    engine.cache.table.check()


def test_state_matters(toy_registered, tmp_path):
    """With the decay at zero the mixer forgets: the two models must differ, so the state is really used."""
    f1 = tb.write_random_model(str(tmp_path / "t1"), CFG, seed=3, std=0.2)
    f0 = tb.write_random_model(str(tmp_path / "t0"), dict(CFG, decay=0.0), seed=3, std=0.2)
    toks = list(range(12))
    outs = []
    for f in (f1, f0):
        e = tb.load(f, dtype="float32", max_tokens=128)
        s = e.open()
        outs.append(e.step([s], [toks], [[11]]).cpu())
    assert float((outs[0] - outs[1]).abs().max()) > 1e-3
