"""A plain, slow implementation of the Llama decoder with a mixture-of-experts feed-forward.

It rests on the formulas of YdrMaster/transformer only: the reference cannot be compiled or
imported here (it is Rust with git dependencies, and its operators live in an external crate), so
no output of the reference anchors this file.  Where the reference delegates a formula to that
external operator crate, the docstring says so and states the form chosen.

Whole sequences, no cache, one function for each part, loops where loops are the clearest.  It
shares no code with the package under test: it reads ``config.json`` and ``model.safetensors`` by
itself and works on CPU tensors in float32 or float64.

File/line citations are paths inside the reference project.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


# ----------------------------------------------------------------------------------------------
# reading a model folder
# ----------------------------------------------------------------------------------------------
def read_folder(folder: str, dtype=torch.float32):
    """config.json as a dict and every tensor of model.safetensors converted to ``dtype``."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name).to(dtype)
    return cfg, tensors


def sizes(cfg: dict) -> dict:
    """The numbers of LlamaMeta (models/llama/common/src/lib.rs:19-40) with the defaults of
    models/llama/common/src/storage.rs:47-59."""
    nh = cfg["num_attention_heads"]
    d = cfg["hidden_size"]
    return dict(
        nblk=cfg["num_hidden_layers"],
        d=d,
        nh=nh,
        nkvh=cfg.get("num_key_value_heads", nh),
        dh=cfg.get("head_dim", d // nh),
        di=cfg["intermediate_size"],
        nexp=cfg.get("num_local_experts", 0),
        nexp_use=cfg.get("num_experts_per_tok", 0),
        nvoc=cfg["vocab_size"],
        eps=cfg.get("rms_norm_eps", 1e-5),
        theta=cfg.get("rope_theta", 1e4),
        tied=cfg.get("tie_word_embeddings", False),
        pairing=cfg.get("rope_pairing", "adjacent"),
    )


# ----------------------------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------------------------
def embedding(token_embd: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x[i] = token_embd[tok_i], no scaling (models/llama/cuda/src/infer.rs:98-104,
    test-utils/src/llama.rs:18-23)."""
    return torch.stack([token_embd[int(t)] for t in tokens])


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * w, per row (call sites models/llama/common/src/compute.rs:207,
    275,362; epsilon passed at :410-422; the arithmetic is in the external operator)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * w


def rope(t: torch.Tensor, positions: Sequence[int], theta: float, pairing: str) -> torch.Tensor:
    """Rotate each head of t [n, heads, dh] by its token's position
    (models/llama/common/src/compute.rs:232-233,457-488: gets pos, sin/cos tables and theta; the
    pairing is inside the external operator).  Angle(p, i) = p * theta^(-2i/dh), i in [0, dh/2).
    "adjacent" rotates (t[2i], t[2i+1]), the form GGUF llama weights are stored for;
    "half" rotates (t[i], t[i + dh/2])."""
    n, heads, dh = t.shape
    half = dh // 2
    out = t.clone()
    for a in range(n):
        p = float(positions[a])
        for i in range(half):
            ang = p * theta ** (-2.0 * i / dh)
            c, s = math.cos(ang), math.sin(ang)
            i0, i1 = (2 * i, 2 * i + 1) if pairing == "adjacent" else (i, i + half)
            x0 = t[a, :, i0]
            x1 = t[a, :, i1]
            out[a, :, i0] = x0 * c - x1 * s
            out[a, :, i1] = x0 * s + x1 * c
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q [n, nh, dh], k and v [n, nkvh, dh] of one whole sequence -> [n, nh, dh].
    Query head h reads key/value head h // (nh / nkvh); the token at position p sees positions
    <= p; scores are scaled by 1/sqrt(dh) (models/llama/common/src/compute.rs:243-264,490-530; scale
    and mask are inside the external operator)."""
    n, nh, dh = q.shape
    nkvh = k.shape[1]
    group = nh // nkvh
    out = torch.zeros_like(q)
    scale = 1.0 / math.sqrt(dh)
    for h in range(nh):
        g = h // group
        for a in range(n):
            s = (k[: a + 1, g] @ q[a, h]) * scale          # [a+1]
            p = torch.softmax(s, dim=0)
            out[a, h] = p @ v[: a + 1, g]
    return out


def _as_stored(store, x: torch.Tensor) -> torch.Tensor:
    """``store`` is the rounding an implementation applies where it writes an activation to memory
    (None: none).  With ``store = lambda x: x.bfloat16().float()`` the functions below predict what a
    bfloat16 path computes, up to the order of its sums; such a path can be compared with that far more
    tightly than with the unrounded result.  Sums, softmax, norms and the residual stream stay as they are."""
    return x if store is None else store(x)


def attention_mixer(x1, w_qkv, w_o, positions, sz, store=None) -> torch.Tensor:
    """qkv = x1 Wqkv^T, split into q heads, k heads, v heads in that order, rope(q), rope(k),
    attention, merge heads, times Wo^T (models/llama/common/src/compute.rs:210-270)."""
    nh, nkvh, dh = sz["nh"], sz["nkvh"], sz["dh"]
    n = x1.shape[0]
    qkv = _as_stored(store, x1 @ w_qkv.T)
    q = qkv[:, : nh * dh].reshape(n, nh, dh)
    k = qkv[:, nh * dh : (nh + nkvh) * dh].reshape(n, nkvh, dh)
    v = qkv[:, (nh + nkvh) * dh :].reshape(n, nkvh, dh)
    q = _as_stored(store, rope(q, positions, sz["theta"], sz["pairing"]))
    k = _as_stored(store, rope(k, positions, sz["theta"], sz["pairing"]))
    o = _as_stored(store, causal_attention(q, k, v).reshape(n, nh * dh))
    return _as_stored(store, o @ w_o.T)


def route(logits: torch.Tensor, k: int):
    """Sort one token's router logits descending, keep the first k, softmax over the kept ones
    (models/llama/common/src/compute.rs:375-394).  Equal logits: the lower expert first."""
    order = sorted(range(logits.numel()), key=lambda e: (-float(logits[e]), e))[:k]
    kept = torch.stack([logits[e] for e in order])
    w = torch.exp(kept - kept[0])
    return order, w / w.sum()


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def expert_ffn(x1_tok, w_gate_up, w_down, store=None) -> torch.Tensor:
    """gate_up = x W_gate_up^T, rows 0..di gate and di..2di up; h = silu(gate) * up; y = h W_down^T
    (models/llama/common/src/compute.rs:320-330)."""
    di = w_down.shape[1]
    gu = w_gate_up @ x1_tok
    return _as_stored(store, w_down @ _as_stored(store, silu(gu[:di]) * gu[di:]))


def moe_feed_forward(x1, w_router, w_gate_up_exps, w_down_exps, k: int, forced=None, margins=None,
                     store=None) -> torch.Tensor:
    """For every token: router logits, top-k with softmax over the kept logits, the weighted sum of
    the kept experts in descending-logit order (models/llama/common/src/compute.rs:294-333).

    Two aids for comparing with an implementation that rounds differently (top-k is discontinuous:
    a near-tie may fall the other way): ``forced[a]`` replaces token a's free choice by a given set
    of experts (weights still from this function's own logits), and ``margins`` collects per token
    (free choice, gap between the k-th and (k+1)-th logit, largest |logit|)."""
    out = torch.zeros_like(x1)
    for a in range(x1.shape[0]):
        logits = w_router @ x1[a]
        experts, weights = route(logits, k)
        if margins is not None:
            srt = sorted((float(v) for v in logits), reverse=True)
            gap = srt[k - 1] - srt[k] if k < len(srt) else float("inf")
            margins.append((list(experts), gap, max(abs(srt[0]), abs(srt[-1]))))
        if forced is not None and set(forced[a]) != set(experts):
            experts = sorted((int(e) for e in forced[a]), key=lambda e: (-float(logits[e]), e))
            kept = torch.stack([logits[e] for e in experts])
            weights = torch.exp(kept - kept[0])
            weights = weights / weights.sum()
        for e, w in zip(experts, weights):
            out[a] += w * expert_ffn(x1[a], w_gate_up_exps[e], w_down_exps[e], store)
    return out


def dense_feed_forward(x1, w_gate_up, w_down, store=None) -> torch.Tensor:
    """The feed-forward of a model without experts (models/llama/common/src/compute.rs:278-292)."""
    return torch.stack([expert_ffn(x1[a], w_gate_up, w_down, store) for a in range(x1.shape[0])])


def block(x, t: Dict[str, torch.Tensor], i: int, positions, sz, forced=None, margins=None, store=None) -> torch.Tensor:
    """x += mixer(norm(x)); x += feed_forward(norm(x)) (models/llama/common/src/compute.rs:204-336)."""
    p = f"blk.{i}."
    x1 = _as_stored(store, rms_norm(x, t[p + "attn_norm.weight"], sz["eps"]))
    x = x + attention_mixer(x1, t[p + "attn_qkv.weight"], t[p + "attn_output.weight"], positions, sz, store)
    x1 = _as_stored(store, rms_norm(x, t[p + "ffn_norm.weight"], sz["eps"]))
    if sz["nexp"] > 0:
        x = x + moe_feed_forward(
            x1,
            t[p + "ffn_gate_inp.weight"],
            t[p + "ffn_gate_up_exps.weight"],
            t[p + "ffn_down_exps.weight"],
            sz["nexp_use"], forced, margins, store,
        )
    else:
        x = x + dense_feed_forward(x1, t[p + "ffn_gate_up.weight"], t[p + "ffn_down.weight"], store)
    return x


def forward(cfg: dict, t: Dict[str, torch.Tensor], tokens: Sequence[int],
            want: Optional[Sequence[int]] = None, forced_routes=None, margins_out=None, store=None) -> torch.Tensor:
    """Logits [len(want), vocab] of one whole sequence that starts at position 0; ``want`` defaults
    to every position.  Final norm and head only on the wanted rows
    (models/llama/common/src/compute.rs:343-365); a missing ``output.weight`` means the head is
    ``token_embd`` (models/llama/common/src/storage.rs:84)."""
    sz = sizes(cfg)
    positions = list(range(len(tokens)))
    x = embedding(t["token_embd.weight"], tokens)
    for i in range(sz["nblk"]):
        # forced_routes[i][a]: experts token a must use in layer i; margins_out[i]: see moe_feed_forward
        m = [] if margins_out is not None else None
        x = block(x, t, i, positions, sz, None if forced_routes is None else forced_routes[i], m, store)
        if margins_out is not None:
            margins_out.append(m)
    rows = list(range(len(tokens))) if want is None else list(want)
    x = _as_stored(store, rms_norm(x[rows], t["output_norm.weight"], sz["eps"]))
    head = t.get("output.weight", t["token_embd.weight"])
    return x @ head.T


# ----------------------------------------------------------------------------------------------
# sampling and generation
# ----------------------------------------------------------------------------------------------
def sample_distribution(logits: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """The distribution the sampler draws from, as (token ids ascending, probabilities).
    temperature 0 means the argmax alone (test-utils/src/lib.rs:78 defaults to 0; the rules are in
    the external operator).  Order of the filters: divide by temperature, keep the top_k largest
    (ties: lower id first), softmax, keep the shortest prefix in descending probability whose mass
    reaches top_p, renormalise."""
    z = logits.to(torch.float64)
    n = z.numel()
    if temperature == 0:
        best = max(range(n), key=lambda i: (float(z[i]), -i))
        return [best], [1.0]
    order = sorted(range(n), key=lambda i: (-float(z[i]), i))
    if top_k and top_k < n:
        order = order[:top_k]
    zz = torch.tensor([float(z[i]) / temperature for i in order], dtype=torch.float64)
    p = torch.softmax(zz, dim=0)
    if top_p < 1.0:
        acc = 0.0
        keep = 0
        for j in range(len(order)):
            acc += float(p[j])
            keep = j + 1
            if acc >= top_p:
                break
        order, p = order[:keep], p[:keep] / p[:keep].sum()
    pairs = sorted(zip(order, p.tolist()))
    return [i for i, _ in pairs], [q for _, q in pairs]


def greedy_generate(cfg, t, prompt: Sequence[int], steps: int, stop: Sequence[int] = ()) -> List[int]:
    """The reference's loop with argmax (test-utils/src/lib.rs:153-173): the stop token ends the
    sequence and is not kept.  Whole-sequence recomputation at every step."""
    seq = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward(cfg, t, seq, want=[len(seq) - 1])[0]
        nxt = int(torch.argmax(logits))
        if nxt in stop:
            break
        out.append(nxt)
        seq.append(nxt)
    return out
