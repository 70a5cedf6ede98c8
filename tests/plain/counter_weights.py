"""The rule for random weights, restated for the tests: element i of tensor ``name`` under ``seed``.

Written from the rule's statement alone (it shares no code with the package), in torch integer
arithmetic so that it runs on the CPU or on a GPU and can produce the tensors of a full-size model
in seconds:

    base  = mix64((seed * G + fnv1a64(name)) mod 2^64)            G = 0x9E3779B97F4A7C15
    h_j   = mix64(base + (2 i + j) * G), j = 0, 1                  mix64: the splitmix64 finalizer
    c     = sum of the eight 16-bit fields of h_0 and h_1, minus 4 * 65535
    value = float32(c) * float32(std / sqrt(8 (2^32 - 1) / 12)), then rounded to the storage type

torch has no unsigned 64-bit arithmetic: int64 products wrap modulo 2^64 all the same, and a logical
right shift is an arithmetic one with the sign's copies masked off.
"""
import math

import numpy as np
import torch

_G = 0x9E3779B97F4A7C15
_M = (1 << 64) - 1


def _signed(z: int) -> int:
    z &= _M
    return z - (1 << 64) if z >= (1 << 63) else z


def _fnv(name: str) -> int:
    h = 0xCBF29CE484222325
    for byte in name.encode():
        h = ((h ^ byte) * 0x100000001B3) & _M
    return h


def _mix_int(z: int) -> int:
    z &= _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def _shr(z: torch.Tensor, n: int) -> torch.Tensor:
    return (z >> n) & ((1 << (64 - n)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _shr(z, 30)) * _signed(0xBF58476D1CE4E5B9)
    z = (z ^ _shr(z, 27)) * _signed(0x94D049BB133111EB)
    return z ^ _shr(z, 31)


def values(seed: int, name: str, shape, std: float, device="cpu", dtype=torch.float32, first: int = 0) -> torch.Tensor:
    """The tensor ``name`` of the given shape as float32 values (rounded through ``dtype`` if that is bfloat16)."""
    n = int(np.prod(shape)) if len(shape) else 1
    base = _signed(_mix_int((seed * _G + _fnv(name)) & _M))
    scale = float(np.float32(std / math.sqrt(8.0 * ((1 << 32) - 1) / 12.0)))
    out = torch.empty(n, dtype=torch.float32, device=device)
    slab = 1 << 24
    for lo in range(0, n, slab):
        m = min(slab, n - lo)
        i2 = torch.arange(first + lo, first + lo + m, dtype=torch.int64, device=device) * 2
        total = torch.zeros(m, dtype=torch.int64, device=device)
        for j in (0, 1):
            h = _mix((i2 + j) * _signed(_G) + base)
            for f in range(4):
                total += _shr(h, 16 * f) & 0xFFFF if f else h & 0xFFFF
        c = (total - 4 * 65535).to(torch.float32)
        out[lo:lo + m] = c * torch.tensor(scale, dtype=torch.float32, device=device)
    if dtype != torch.float32:
        out = out.to(dtype).to(torch.float32)
    return out.view(*shape)


def llama_tensors(cfg: dict, seed: int, std: float, device="cpu", dtype=torch.float32, layers=None) -> dict:
    """Every tensor of a Llama(-MoE) model with random weights, under the names the reference reads
    (models/llama/common/src/storage.rs:32-34,63-84); norm weights are one.  ``layers``: only these blocks
    (plus the embedding, the final norm and the head), for a caller that walks a large model block by block."""
    d, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    nkvh, dh = cfg.get("num_key_value_heads", nh), cfg.get("head_dim", d // nh)
    di, E, V = cfg["intermediate_size"], cfg.get("num_local_experts", 0), cfg["vocab_size"]

    def rnd(name, *shape):
        return values(seed, name, shape, std, device, dtype)

    t = {}
    if layers is None or "ends" in layers:
        t["token_embd.weight"] = rnd("token_embd.weight", V, d)
        t["output_norm.weight"] = torch.ones(d, device=device)
        if not cfg.get("tie_word_embeddings", False):
            t["output.weight"] = rnd("output.weight", V, d)
    for i in range(cfg["num_hidden_layers"]):
        if layers is not None and i not in layers:
            continue
        p = f"blk.{i}."
        t[p + "attn_norm.weight"] = torch.ones(d, device=device)
        t[p + "ffn_norm.weight"] = torch.ones(d, device=device)
        t[p + "attn_qkv.weight"] = rnd(p + "attn_qkv.weight", (nh + 2 * nkvh) * dh, d)
        t[p + "attn_output.weight"] = rnd(p + "attn_output.weight", d, nh * dh)
        if E:
            t[p + "ffn_gate_inp.weight"] = rnd(p + "ffn_gate_inp.weight", E, d)
            t[p + "ffn_gate_up_exps.weight"] = rnd(p + "ffn_gate_up_exps.weight", E, 2 * di, d)
            t[p + "ffn_down_exps.weight"] = rnd(p + "ffn_down_exps.weight", E, d, di)
        else:
            t[p + "ffn_gate_up.weight"] = rnd(p + "ffn_gate_up.weight", 2 * di, d)
            t[p + "ffn_down.weight"] = rnd(p + "ffn_down.weight", d, di)
    return t
