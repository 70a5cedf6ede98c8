"""The Llama decoder, with a mixture-of-experts feed-forward when the configuration has experts.

Everything that is particular to this architecture lives in this file: how its configuration
becomes a :class:`ModelSpec`, and which file tensors fill which parameters.  Tensor names are the
ones the reference reads (models/llama/common/src/storage.rs:32-34,63-84):

    token_embd.weight [nvoc, d]          output_norm.weight [d]       output.weight [nvoc, d] (optional)
    blk.N.attn_norm.weight [d]           blk.N.attn_qkv.weight [(nh + 2 nkvh) dh, d]   (rows q, k, v)
    blk.N.attn_output.weight [d, nh dh]  blk.N.ffn_norm.weight [d]
    blk.N.ffn_gate_inp.weight [nexp, d]
    blk.N.ffn_gate_up_exps.weight [nexp, 2 di, d]  (per expert: gate rows, then up rows)
    blk.N.ffn_down_exps.weight [nexp, d, di]
    dense (nexp = 0): blk.N.ffn_gate_up.weight [2 di, d], blk.N.ffn_down.weight [d, di]

The reference expects q/k/v and gate/up already merged by an external tool
(docs/user-guide/doc.md:128-140).  Files that still hold them apart (blk.N.attn_q / attn_k /
attn_v, blk.N.ffn_gate_exps / ffn_up_exps, blk.N.ffn_gate / ffn_up) are accepted and merged here.
"""
from __future__ import annotations

from typing import List

from ..config.llama import LlamaMeta
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..weights.plan import Source, TensorRule, single


def build_spec(m: LlamaMeta) -> ModelSpec:
    norm = PartSpec.of("rmsnorm", width=m.d, eps=m.epsilon)
    rope = PartSpec.of("rope", dh=m.dh, theta=m.theta, pairing=m.rope_pairing, positions=m.nctx)
    mixer = PartSpec.of("attention", width=m.d, nh=m.nh, nkvh=m.nkvh, dh=m.dh, position=rope)
    if m.is_moe:
        ff = PartSpec.of("moe", width=m.d, di=m.di, nexp=m.nexp, nexp_use=m.nexp_use)
    else:
        ff = PartSpec.of("swiglu", width=m.d, di=m.di)
    layer = LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm)
    return ModelSpec(
        width=m.d, vocab=m.nvoc, max_context=m.nctx,
        layers=tuple(layer for _ in range(m.nblk)),
        order=tuple(RunEntry(i) for i in range(m.nblk)),
        embedding=PartSpec.of("lookup", vocab=m.nvoc, width=m.d),
        final_norm=norm,
        head=PartSpec.of("linear", vocab=m.nvoc, width=m.d, tied=m.tied),
        stop_tokens=tuple(m.eos),
    )


def tensor_plan(m: LlamaMeta) -> List[TensorRule]:
    d, dh, di, E = m.d, m.dh, m.di, m.nexp
    q, kv = m.nh * dh, m.nkvh * dh
    rules = [TensorRule(("embedding", "table"), (m.nvoc, d), "matrix", (single("token_embd.weight", (m.nvoc, d)),))]
    for i in range(m.nblk):
        p = f"blk.{i}."
        L = ("layers", i)
        rules.append(TensorRule(L + ("mixer_norm", "weight"), (d,), "norm",
                                (single(p + "attn_norm.weight", (d,)),), init="ones"))
        rules.append(TensorRule(L + ("mixer", "wqkv"), (q + 2 * kv, d), "matrix", (
            single(p + "attn_qkv.weight", (q + 2 * kv, d)),
            Source((p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"), ((q, d), (kv, d), (kv, d)), "cat0"),
        )))
        rules.append(TensorRule(L + ("mixer", "wo"), (d, q), "matrix", (single(p + "attn_output.weight", (d, q)),)))
        rules.append(TensorRule(L + ("feed_forward_norm", "weight"), (d,), "norm",
                                (single(p + "ffn_norm.weight", (d,)),), init="ones"))
        if m.is_moe:
            rules.append(TensorRule(L + ("feed_forward", "router"), (E, d), "matrix",
                                    (single(p + "ffn_gate_inp.weight", (E, d)),)))
            rules.append(TensorRule(L + ("feed_forward", "wgu"), (E, 2 * di, d), "matrix", (
                single(p + "ffn_gate_up_exps.weight", (E, 2 * di, d)),
                Source((p + "ffn_gate_exps.weight", p + "ffn_up_exps.weight"), ((E, di, d), (E, di, d)), "cat1"),
                # one matrix per expert (files written before the experts were stacked): blk.N.ffn_gate.E.weight, ...
                Source(tuple(p + f"ffn_{which}.{e}.weight" for e in range(E) for which in ("gate", "up")),
                       ((di, d),) * (2 * E), "stack0_of_row_pairs"),
            )))
            rules.append(TensorRule(L + ("feed_forward", "wd"), (E, d, di), "matrix", (
                single(p + "ffn_down_exps.weight", (E, d, di)),
                Source(tuple(p + f"ffn_down.{e}.weight" for e in range(E)), ((d, di),) * E, "stack0"),
            )))
        else:
            rules.append(TensorRule(L + ("feed_forward", "wgu"), (2 * di, d), "matrix", (
                single(p + "ffn_gate_up.weight", (2 * di, d)),
                Source((p + "ffn_gate.weight", p + "ffn_up.weight"), ((di, d), (di, d)), "cat0"),
            )))
            rules.append(TensorRule(L + ("feed_forward", "wd"), (d, di), "matrix",
                                    (single(p + "ffn_down.weight", (d, di)),)))
    rules.append(TensorRule(("final_norm", "weight"), (d,), "norm", (single("output_norm.weight", (d,)),), init="ones"))
    if m.tied:
        # no tensor of its own is required; one that is present is still read (storage.rs:84)
        rules.append(TensorRule(("head", "weight"), (m.nvoc, d), "matrix", (single("output.weight", (m.nvoc, d)),),
                                shared_with=("embedding", "table")))
    else:
        rules.append(TensorRule(("head", "weight"), (m.nvoc, d), "matrix", (single("output.weight", (m.nvoc, d)),)))
    return rules


LLAMA = register_architecture(Architecture(
    name="llama",
    config_cls=LlamaMeta,
    build_spec=build_spec,
    tensor_plan=tensor_plan,
    names=("llama", "llama_moe", "LlamaMoe", "Llama", "LlamaForCausalLM", "LlamaMoEForCausalLM"),
))
