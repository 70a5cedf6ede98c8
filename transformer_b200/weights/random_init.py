"""Random weights from a configuration and a seed.

The reference has no such mode (it only reads converted GGUF files).  Norm weights are one.  Every
other value is a function of (seed, the tensor's name in the file, the element's index): see
:mod:`.counter_random`.  So the folder written on the CPU, the weights filled on the GPU and a test's
own restatement of the rule hold the same bits, whoever computes them and in which order.

* :func:`write_model_folder` writes ``config.json`` and ``model.safetensors`` (computed on the CPU).
* :func:`random_device_weights` fills the parameters directly on the GPU, by the fill kernel, for
  models too large to be worth a file: the same values as the folder's.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Sequence

import torch
from safetensors.torch import save_file

from . import counter_random
from .loader import storage_dtype
from .plan import Dest, TensorRule


def _canonical_name(rule: TensorRule) -> str:
    src = rule.canonical
    if len(src.names) != 1:
        raise ValueError(f"the canonical source of {rule.dest} must be one tensor")
    return src.names[0]


def _host_tensor(rule: TensorRule, seed: int, std: float) -> torch.Tensor:
    shape = rule.canonical.shapes[0]
    if rule.init == "ones":
        return torch.ones(shape, dtype=torch.float32)
    if rule.init == "normal":
        n = 1
        for s in shape:
            n *= int(s)
        return torch.from_numpy(counter_random.normal_values(seed, _canonical_name(rule), 0, n, std)).view(*shape)
    raise ValueError(f"unknown init {rule.init!r}")


def random_file_tensors(rules: Sequence[TensorRule], seed: int, matrix_dtype: torch.dtype,
                        std: float = 0.02) -> Dict[str, torch.Tensor]:
    """{file tensor name: CPU tensor} for the canonical source of every rule that owns storage."""
    out: Dict[str, torch.Tensor] = {}
    for rule in rules:
        if rule.shared_with is not None:
            continue   # tied: the file holds no tensor of its own
        t = _host_tensor(rule, int(seed), std)
        out[_canonical_name(rule)] = t.to(storage_dtype(rule.role, matrix_dtype)).contiguous()
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
    """The parameters on the device, each filled in place by the counter-based kernel: no staging copy, and
    the same values that :func:`write_model_folder` would have put into a file."""
    from ..csrc import lib
    out: Dict[Dest, torch.Tensor] = {}
    with torch.cuda.device(device):
        for rule in rules:
            if rule.shared_with is not None:
                continue
            dtype = storage_dtype(rule.role, compute_dtype)
            if rule.init == "ones":
                out[rule.dest] = torch.ones(rule.shape, dtype=dtype, device=device)
                continue
            if rule.init != "normal":
                raise ValueError(f"unknown init {rule.init!r}")
            if tuple(rule.canonical.shapes[0]) != tuple(rule.shape):
                raise ValueError(f"{rule.dest}: the canonical file tensor and the parameter differ in shape")
            t = torch.empty(rule.shape, dtype=dtype, device=device)
            lib.random_fill(t, counter_random.stream_base(seed, _canonical_name(rule)),
                            float(counter_random.scale_for(std)))
            out[rule.dest] = t
    for rule in rules:
        if rule.shared_with is not None:
            out[rule.dest] = out[rule.shared_with]
    return out
