"""The plain implementation once more, without its loops over tokens and heads.

``llama_moe_plain`` states every formula with a loop where a loop is the clearest; that makes a
model of 32 layers of width 4096 unaffordable.  This file states the same formulas on whole tensors
(a test pins the two to each other on the tiny configurations in float64), so that the engine can be
checked at the benchmark's own depth.  Same rules as there: whole sequences, no cache, one function
for each part, no code shared with the package, tensors on whatever device and in whatever float
type the caller hands in (float64 is the yardstick).  Citations are paths inside the reference.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch


def sizes(cfg: dict) -> dict:
    """LlamaMeta's numbers (models/llama/common/src/lib.rs:19-40, defaults storage.rs:47-59)."""
    nh, d = cfg["num_attention_heads"], cfg["hidden_size"]
    return dict(nblk=cfg["num_hidden_layers"], d=d, nh=nh, nkvh=cfg.get("num_key_value_heads", nh),
                dh=cfg.get("head_dim", d // nh), di=cfg["intermediate_size"], nexp=cfg.get("num_local_experts", 0),
                nexp_use=cfg.get("num_experts_per_tok", 0), eps=cfg.get("rms_norm_eps", 1e-5),
                theta=cfg.get("rope_theta", 1e4), pairing=cfg.get("rope_pairing", "adjacent"))


def _st(store, x):
    """Round where an implementation stores an activation (see llama_moe_plain._as_stored)."""
    return x if store is None else store(x)


def embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """x[i] = token_embd[tok_i] (models/llama/cuda/src/infer.rs:98-104)."""
    return table[tokens]


def rms_norm(x, w, eps):
    """y = x / sqrt(mean(x^2) + eps) * w (models/llama/common/src/compute.rs:207,275,362)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rope(t: torch.Tensor, positions: torch.Tensor, theta: float, pairing: str) -> torch.Tensor:
    """t [n, heads, dh] rotated by angle(p, i) = p * theta^(-2i/dh); pairs (2i, 2i+1) when "adjacent",
    (i, i + dh/2) when "half" (models/llama/common/src/compute.rs:232-233,457-488).  Angles in float64."""
    n, heads, dh = t.shape
    half = dh // 2
    i = torch.arange(half, dtype=torch.float64, device=t.device)
    ang = positions.to(torch.float64)[:, None] * torch.pow(torch.tensor(theta, dtype=torch.float64, device=t.device),
                                                            -2.0 * i / dh)[None, :]
    c, s = torch.cos(ang).to(t.dtype)[:, None, :], torch.sin(ang).to(t.dtype)[:, None, :]
    if pairing == "adjacent":
        x0, x1 = t[..., 0::2], t[..., 1::2]
        out = torch.empty_like(t)
        out[..., 0::2] = x0 * c - x1 * s
        out[..., 1::2] = x0 * s + x1 * c
        return out
    x0, x1 = t[..., :half], t[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def causal_attention(q, k, v):
    """q [n, nh, dh]; k, v [n, nkvh, dh] -> [n, nh, dh]; head h reads key/value head h // (nh / nkvh); position p
    sees positions <= p; scores scaled by 1/sqrt(dh) (models/llama/common/src/compute.rs:243-264,490-530)."""
    n, nh, dh = q.shape
    group = nh // k.shape[1]
    kk = k.repeat_interleave(group, dim=1).transpose(0, 1)        # [nh, n, dh]
    vv = v.repeat_interleave(group, dim=1).transpose(0, 1)
    out = torch.empty_like(q)
    mask = torch.ones((n, n), dtype=torch.bool, device=q.device).tril()
    for h0 in range(0, nh, 8):            # a few heads at a time: the score matrix of all heads may be large
        qq = q[:, h0:h0 + 8].transpose(0, 1)
        s = qq @ kk[h0:h0 + 8].transpose(1, 2) / math.sqrt(dh)
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h0:h0 + 8] = (torch.softmax(s, dim=-1) @ vv[h0:h0 + 8]).transpose(0, 1)
    return out


def attention_mixer(x1, w_qkv, w_o, positions, sz, store=None):
    """qkv = x1 Wqkv^T, heads in the order q, k, v; rope(q), rope(k); attention; times Wo^T
    (models/llama/common/src/compute.rs:210-270)."""
    nh, nkvh, dh = sz["nh"], sz["nkvh"], sz["dh"]
    n = x1.shape[0]
    qkv = _st(store, x1 @ w_qkv.T)
    q = qkv[:, :nh * dh].reshape(n, nh, dh)
    k = qkv[:, nh * dh:(nh + nkvh) * dh].reshape(n, nkvh, dh)
    v = qkv[:, (nh + nkvh) * dh:].reshape(n, nkvh, dh)
    q = _st(store, rope(q, positions, sz["theta"], sz["pairing"]))
    k = _st(store, rope(k, positions, sz["theta"], sz["pairing"]))
    o = _st(store, causal_attention(q, k, v).reshape(n, nh * dh))
    return _st(store, o @ w_o.T)


def route(logits: torch.Tensor, k: int):
    """Per token: experts by descending logit, equal logits to the lower expert, the first k kept, softmax over
    the kept logits (models/llama/common/src/compute.rs:375-394).  Returns (experts [n, k], weights [n, k])."""
    order = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :k]
    kept = torch.gather(logits, 1, order)
    w = torch.exp(kept - kept[:, :1])
    return order, w / w.sum(dim=-1, keepdim=True)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def moe_feed_forward(x1, w_router, w_gu, w_d, k, forced=None, margins=None, store=None):
    """Router, top-k, every kept expert's SwiGLU, and their weighted sum in descending-logit order
    (models/llama/common/src/compute.rs:294-333).  ``forced`` [n, k] replaces the free choice of the tokens whose
    set of experts differs from it (weights still from this function's logits); ``margins`` receives, per token,
    (free choice, gap between the k-th and (k+1)-th logit, largest |logit|)."""
    n, E = x1.shape[0], w_router.shape[0]
    di = w_d.shape[2]
    logits = x1 @ w_router.T
    experts, weights = route(logits, k)
    if margins is not None:
        srt = torch.sort(logits, dim=-1, descending=True).values
        gap = srt[:, k - 1] - srt[:, k] if k < E else torch.full((n,), float("inf"), device=x1.device)
        big = logits.abs().max(dim=-1).values
        margins.extend((experts[a].tolist(), float(gap[a]), float(big[a])) for a in range(n))
    if forced is not None:
        forced = torch.as_tensor(forced, device=x1.device, dtype=torch.long)
        differs = (torch.sort(forced, dim=-1).values != torch.sort(experts, dim=-1).values).any(dim=-1)
        if bool(differs.any()):
            fl = torch.gather(logits, 1, forced)
            # descending logit, equal logits to the lower expert: sort by expert first, then stably by logit
            by_e = torch.sort(forced, dim=-1)
            fl = torch.gather(fl, 1, by_e.indices)
            by_l = torch.sort(fl, dim=-1, descending=True, stable=True)
            f_exp = torch.gather(by_e.values, 1, by_l.indices)
            f_w = torch.exp(by_l.values - by_l.values[:, :1])
            f_w = f_w / f_w.sum(dim=-1, keepdim=True)
            experts = torch.where(differs[:, None], f_exp, experts)
            weights = torch.where(differs[:, None], f_w, weights)
    y = torch.zeros((n, k, x1.shape[1]), dtype=x1.dtype, device=x1.device)
    for e in range(E):
        tok, rank = torch.nonzero(experts == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        gu = x1[tok] @ w_gu[e].T
        h = _st(store, silu(gu[:, :di]) * gu[:, di:])
        y[tok, rank] = _st(store, h @ w_d[e].T)
    out = torch.zeros_like(x1)
    for j in range(k):                     # the reference adds one expert after the other, best first
        out = out + weights[:, j:j + 1] * y[:, j]
    return out


def dense_feed_forward(x1, w_gu, w_d, store=None):
    """models/llama/common/src/compute.rs:278-292."""
    di = w_d.shape[1]
    gu = x1 @ w_gu.T
    return _st(store, _st(store, silu(gu[:, :di]) * gu[:, di:]) @ w_d.T)


def block(x, t: Dict[str, torch.Tensor], i: int, positions, sz, forced=None, margins=None, store=None):
    """x += mixer(norm(x)); x += feed_forward(norm(x)) (models/llama/common/src/compute.rs:204-336)."""
    p = f"blk.{i}."
    x1 = _st(store, rms_norm(x, t[p + "attn_norm.weight"], sz["eps"]))
    x = x + attention_mixer(x1, t[p + "attn_qkv.weight"], t[p + "attn_output.weight"], positions, sz, store)
    x1 = _st(store, rms_norm(x, t[p + "ffn_norm.weight"], sz["eps"]))
    if sz["nexp"] > 0:
        return x + moe_feed_forward(x1, t[p + "ffn_gate_inp.weight"], t[p + "ffn_gate_up_exps.weight"],
                                    t[p + "ffn_down_exps.weight"], sz["nexp_use"], forced, margins, store)
    return x + dense_feed_forward(x1, t[p + "ffn_gate_up.weight"], t[p + "ffn_down.weight"], store)


def head(x, t, rows, sz, store=None):
    """Final norm and lm_head on the wanted rows only (models/llama/common/src/compute.rs:343-365); a missing
    ``output.weight`` means the head is ``token_embd`` (storage.rs:84)."""
    xr = _st(store, rms_norm(x[rows], t["output_norm.weight"], sz["eps"]))
    return xr @ t.get("output.weight", t["token_embd.weight"]).T


def forward_many(cfg: dict, t, requests: Sequence[Sequence[int]], wants=None, forced_routes=None, margins_out=None,
                 store=None, tensors_of_layer=None):
    """:func:`forward` for several independent sequences, block by block for all of them: a model whose blocks are
    produced on demand (``tensors_of_layer(i)``; ``t`` then holds the embedding, the final norm and the head) is
    walked once.  forced_routes[r][i] / margins_out[r][i] belong to request r, block i.  Returns a list of logits."""
    sz = sizes(cfg)
    ref = t["token_embd.weight"]
    xs, poss = [], []
    for tokens in requests:
        tok = torch.as_tensor(list(tokens), dtype=torch.long, device=ref.device)
        xs.append(embedding(ref, tok))
        poss.append(torch.arange(len(tokens), device=ref.device))
    if margins_out is not None:
        margins_out.extend([] for _ in requests)
    for i in range(sz["nblk"]):
        ti = t if tensors_of_layer is None else tensors_of_layer(i)
        for r in range(len(requests)):
            m = [] if margins_out is not None else None
            forced = None if forced_routes is None or forced_routes[r] is None else forced_routes[r][i]
            xs[r] = block(xs[r], ti, i, poss[r], sz, forced, m, store)
            if margins_out is not None:
                margins_out[r].append(m)
        del ti
    out = []
    for r, tokens in enumerate(requests):
        rows = list(range(len(tokens))) if wants is None or wants[r] is None else list(wants[r])
        out.append(head(xs[r], t, torch.as_tensor(rows, dtype=torch.long, device=ref.device), sz, store))
    return out


def forward(cfg: dict, t, tokens: Sequence[int], want: Optional[Sequence[int]] = None, forced_routes=None,
            margins_out=None, store=None, tensors_of_layer=None) -> torch.Tensor:
    """Logits [len(want), vocab] of one whole sequence from position 0; ``want`` defaults to every position."""
    m = [] if margins_out is not None else None
    out = forward_many(cfg, t, [tokens], [want], None if forced_routes is None else [forced_routes], m, store,
                       tensors_of_layer)
    if margins_out is not None:
        margins_out.extend(m[0])
    return out[0]
