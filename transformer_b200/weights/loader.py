"""Weights from ``model.safetensors`` by tensor name.

The reference reads tensors by exact name and panics on the first absent one
(gguf/src/lib.rs:160-164, models/llama/common/src/storage.rs:32-34,63-78).  Here every fault of a
file is gathered first and reported in ONE error: missing tensors, unexpected tensors and wrong
shapes, each listed.  Nothing is uploaded before the file is known to be whole.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, Iterable, List, Mapping, Sequence, Tuple

import torch
from safetensors import safe_open

from .plan import Dest, Source, TensorRule


class WeightError(RuntimeError):
    """One error for everything that is wrong with a weight file."""

    def __init__(self, path: str, missing=(), unexpected=(), wrong_shape=(), wrong_type=()):
        self.path = path
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)   # (name, found, expected)
        self.wrong_type = list(wrong_type)     # (name, found dtype, role)
        lines = [f"weights in {path} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(f)}, expected {list(e)}" for n, f, e in self.wrong_shape))
        if self.wrong_type:
            lines.append(f"  unsupported types ({len(self.wrong_type)}): " + ", ".join(
                f"{n} is {t} but is a {r}" for n, t, r in self.wrong_type))
        super().__init__("\n".join(lines))


def storage_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "matrix":
        return compute_dtype
    if role == "norm":
        return torch.float32
    if role == "table":
        return torch.int32
    raise ValueError(f"unknown tensor role {role!r}")


class _Files:
    """All ``*.safetensors`` files of a folder (or one file) as one name -> tensor mapping."""

    def __init__(self, path: str):
        if os.path.isdir(path):
            files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
            if not files:
                raise FileNotFoundError(f"no .safetensors file in {path}")
        else:
            files = [path]
        self.path = path
        self.handles = [safe_open(f, framework="pt", device="cpu") for f in files]
        self.where: Dict[str, int] = {}
        for i, h in enumerate(self.handles):
            for name in h.keys():
                if name in self.where:
                    raise WeightError(path, unexpected=[f"{name} (stored twice)"])
                self.where[name] = i

    def names(self) -> Iterable[str]:
        return self.where.keys()

    def shape_dtype(self, name: str):
        sl = self.handles[self.where[name]].get_slice(name)
        return tuple(sl.get_shape()), sl.get_dtype()

    def tensor(self, name: str) -> torch.Tensor:
        return self.handles[self.where[name]].get_tensor(name)


def check_rules(rules: Sequence[TensorRule], present: Mapping[str, Tuple[Tuple[int, ...], str]], path: str):
    """Choose a source for every rule or raise the one error.  ``present`` maps each tensor name
    of the file to (shape, dtype string).  Returns {dest: Source or None (shared)}."""
    chosen: Dict[Dest, Source] = {}
    used = set()
    missing: List[str] = []
    wrong_shape = []
    wrong_type = []
    for rule in rules:
        pick = None
        for src in rule.sources:
            if all(n in present for n in src.names):
                pick = src
                break
        if pick is None:
            # a partly present alternative counts as the one meant: report what it lacks
            partial = [s for s in rule.sources if any(n in present for n in s.names)]
            if partial:
                src = partial[0]
                used.update(n for n in src.names if n in present)
                missing.extend(n for n in src.names if n not in present)
            elif rule.shared_with is not None:
                chosen[rule.dest] = None
            else:
                missing.extend(rule.canonical.names)
            continue
        chosen[rule.dest] = pick
        for n, want in zip(pick.names, pick.shapes):
            used.add(n)
            shape, dt = present[n]
            if tuple(shape) != tuple(want):
                wrong_shape.append((n, tuple(shape), tuple(want)))
            is_int = dt.upper().startswith(("I", "U")) or dt.upper() == "BOOL"
            plain = dt.upper() in ("F32", "F16", "BF16", "F64")
            if (rule.role == "table") != is_int or (not is_int and not plain):
                wrong_type.append((n, dt, rule.role))
    unexpected = sorted(n for n in present if n not in used)
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(path, missing, unexpected, wrong_shape, wrong_type)
    return chosen


def open_tensors(path: str):
    """The tensors of a model: a folder or file of safetensors, or a GGUF file (any shard of a sharded one)."""
    if os.path.isfile(path) and path.endswith(".gguf"):
        from .gguf import open_gguf
        return open_gguf(path)
    return _Files(path)


def load_weights(path: str, rules: Sequence[TensorRule], compute_dtype: torch.dtype,
                 device: torch.device) -> Dict[Dest, torch.Tensor]:
    """Read, check, convert and upload.  Returns {dest: device tensor}; a rule without a source in
    the file shares the tensor of ``shared_with``."""
    files = open_tensors(path)
    present = {n: files.shape_dtype(n) for n in files.names()}
    chosen = check_rules(rules, present, path)
    out: Dict[Dest, torch.Tensor] = {}
    for rule in rules:
        src = chosen[rule.dest]
        if src is None:
            continue
        parts = [files.tensor(n) for n in src.names]
        t = src.combine(parts)
        t = t.to(storage_dtype(rule.role, compute_dtype)).contiguous()
        out[rule.dest] = t.to(device, non_blocking=False)
    for rule in rules:
        if chosen[rule.dest] is None:
            out[rule.dest] = out[rule.shared_with]
    return out
