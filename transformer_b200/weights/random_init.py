"""Random weights from a configuration and a seed.

The reference has no such mode (it only reads converted GGUF files).  Matrices are drawn from
N(0, std) in float32 and then rounded to the storage type; norm weights are one.  Tensors are drawn
one by one in the order of the tensor plan from ONE generator, so the same plan and seed always
give the same folder.

* :func:`write_model_folder` writes ``config.json`` and ``model.safetensors`` (drawn on the CPU).
* :func:`random_device_weights` fills the parameters directly on the GPU for models too large to
  be worth a file (its values differ from the folder's: another generator).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Sequence

import torch
from safetensors.torch import save_file

from .loader import storage_dtype
from .plan import Dest, TensorRule


def _draw(shape, init: str, std: float, gen: torch.Generator, device) -> torch.Tensor:
    if init == "ones":
        return torch.ones(shape, dtype=torch.float32, device=device)
    if init == "normal":
        return torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * std
    raise ValueError(f"unknown init {init!r}")


def random_file_tensors(rules: Sequence[TensorRule], seed: int, matrix_dtype: torch.dtype,
                        std: float = 0.02) -> Dict[str, torch.Tensor]:
    """{file tensor name: CPU tensor} for the canonical source of every rule that owns storage."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for rule in rules:
        if rule.shared_with is not None:
            continue   # tied: the file holds no tensor of its own
        src = rule.canonical
        if len(src.names) != 1:
            raise ValueError(f"the canonical source of {rule.dest} must be one tensor")
        t = _draw(src.shapes[0], rule.init, std, gen, "cpu")
        out[src.names[0]] = t.to(storage_dtype(rule.role, matrix_dtype)).contiguous()
    return out


def write_model_folder(folder: str, config: Mapping, rules: Sequence[TensorRule], seed: int,
                       matrix_dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> str:
    os.makedirs(folder, exist_ok=True)
    tensors = random_file_tensors(rules, seed, matrix_dtype, std)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(config), f, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return folder


def random_device_weights(rules: Sequence[TensorRule], seed: int, compute_dtype: torch.dtype,
                          device: torch.device, std: float = 0.02) -> Dict[Dest, torch.Tensor]:
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out: Dict[Dest, torch.Tensor] = {}
    for rule in rules:
        if rule.shared_with is not None:
            continue
        # large matrices are drawn in row slabs so the float32 staging copy stays small
        dtype = storage_dtype(rule.role, compute_dtype)
        t = torch.empty(rule.shape, dtype=dtype, device=device)
        flat = t.view(-1)
        step = 1 << 26
        for lo in range(0, flat.numel(), step):
            n = min(step, flat.numel() - lo)
            flat[lo:lo + n] = _draw((n,), rule.init, std, gen, device).to(dtype)
        out[rule.dest] = t
    for rule in rules:
        if rule.shared_with is not None:
            out[rule.dest] = out[rule.shared_with]
    return out
