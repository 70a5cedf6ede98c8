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
    """All of the step's numbers come from the device arrays of ``ctx`` (slots, positions, which sequence a token
    belongs to), never from the host lists, and nothing branches on a value: the forward pass can be captured into
    a CUDA graph and replayed for other slots, which ``graph_safe`` declares."""
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d, self.decay = int(params["width"]), float(params["decay"])

    def parameters(self):
        return {"w": ParamDecl((self.d, self.d))}

    def state_need(self):
        return StateNeed((self.d,), torch.float32)

    def forward(self, ctx, x1, out, cache, state):
        assert cache is None and state is not None
        seq, pos = ctx.tok_seq.long(), ctx.tok_pos.long()             # per token, on the device
        slots = ctx.slots.long()                                      # per sequence
        since = (pos - ctx.seq_pos0.long()[seq] + 1).double()         # tokens of its sequence up to and with this one
        # s_i = decay^since_i * s_before + sum over earlier tokens m of the same sequence of decay^(pos_i - pos_m) x_m
        same = (seq[:, None] == seq[None, :]) & (pos[:, None] >= pos[None, :])
        # (a scalar base keeps torch.pow on the device: a tensor made from a Python number would be copied from
        # the host, which a graph capture refuses)
        weight = torch.pow(self.decay, (pos[:, None] - pos[None, :]).clamp(min=0).double()) * same
        s = weight.float() @ x1.float() + torch.pow(self.decay, since).float()[:, None] * state[slots][seq]
        last = ctx.seq_start.long()[1:] - 1                           # each sequence's last token of the step
        state.index_copy_(0, slots, s[last])
        out.copy_((s @ self.weights["w"].float().T).to(out.dtype))


class RunningSumOnTheHost(RunningSum):
    """The same mixer written the easy way: it walks the host lists.  A captured graph would replay it with the
    slot numbers of the step that was captured, so it must not say ``graph_safe`` (the default is False), and the
    engine then keeps the whole model on eager steps."""
    graph_safe = False

    def forward(self, ctx, x1, out, cache, state):
        w = self.weights["w"].float()
        lo = 0
        for b, n in enumerate(ctx.h_lens):
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


def _decode(engine, prompts, feeds, slots_first=()):
    """Open slots (after some that are only held to shift the numbering), prompts together, then one token each."""
    held = [engine.open() for _ in slots_first]
    slots = [engine.open() for _ in prompts]
    engine.step(slots, prompts)
    outs = [engine.step(slots, [[f[j]] for f in feeds]).cpu().clone() for j in range(len(feeds[0]))]
    for s in slots + held:
        engine.close(s)
    return slots, outs


def test_a_captured_batch_size_is_replayed_with_other_slots(toy_registered, tmp_path):
    """The toy model says graph_safe, so its decode steps are captured.  The graph of batch size 2 is captured
    with slots 0 and 1 and then replayed for sequences in slots 3 and 4 and in slots 1 and 0: the logits are those of
    eager steps, bit for bit.  A part that read ``ctx.h_slots`` would have been replayed with slots 0 and 1."""
    folder = tb.write_random_model(str(tmp_path / "toy"), CFG, seed=3, std=0.2)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 50, (n,), generator=g).tolist() for n in (7, 3)]
    feeds = [torch.randint(0, 50, (6,), generator=g).tolist() for _ in range(2)]
    eager = tb.load(folder, dtype="float32", max_tokens=512)
    eager.use_graphs = False
    _, want = _decode(eager, prompts, feeds)
    engine = tb.load(folder, dtype="float32", max_tokens=512)
    assert engine.graph_safe
    slots, got = _decode(engine, prompts, feeds)
    assert slots == [0, 1] and 2 in engine._graphs
    graph = engine._graphs[2][0]
    slots, moved = _decode(engine, prompts, feeds, slots_first=(0, 1, 2))
    assert slots == [3, 4] and engine._graphs[2][0] is graph, "the same captured graph, other slots"
    _, swapped = _decode(engine, prompts[::-1], feeds[::-1])
    for a, b, c, d in zip(want, got, moved, swapped):
        assert torch.equal(a, b) and torch.equal(a, c) and torch.equal(a, d.flip(0))


def test_a_part_that_walks_host_lists_keeps_the_model_on_eager_steps(tmp_path):
    MIXERS.register("running_sum", RunningSumOnTheHost)
    register_architecture(Architecture("toy_running_sum", ToyConfig, toy_spec, lambda c: plan_from_spec(toy_spec(c))))
    try:
        folder = tb.write_random_model(str(tmp_path / "toy"), CFG, seed=3, std=0.2)
        g = torch.Generator().manual_seed(4)
        prompts = [torch.randint(0, 50, (n,), generator=g).tolist() for n in (7, 3)]
        feeds = [torch.randint(0, 50, (6,), generator=g).tolist() for _ in range(2)]
        engine = tb.load(folder, dtype="float32", max_tokens=512)
        assert not engine.graph_safe and engine.use_graphs
        _, first = _decode(engine, prompts, feeds)
        _, moved = _decode(engine, prompts, feeds, slots_first=(0, 1, 2))
        assert not engine._graphs, "nothing may be captured"
        for a, b in zip(first, moved):
            assert torch.equal(a, b)
        out = tb.generate(engine, prompts, max_steps=4, stop_tokens=()).tokens      # device-fed steps, still eager
        assert [len(t) for t in out] == [4, 4]
    finally:
        unregister_architecture("toy_running_sum")
        MIXERS.unregister("running_sum")
    # and the device form computes the same thing as the easy form
    MIXERS.register("running_sum", RunningSum)
    register_architecture(Architecture("toy_running_sum", ToyConfig, toy_spec, lambda c: plan_from_spec(toy_spec(c))))
    try:
        engine = tb.load(folder, dtype="float32", max_tokens=512)
        _, device_form = _decode(engine, prompts, feeds)
    finally:
        unregister_architecture("toy_running_sum")
        MIXERS.unregister("running_sum")
    for a, b in zip(first, device_form):
        assert float((a - b).abs().max()) <= 2e-4


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
