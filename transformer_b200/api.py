"""The entry points a user calls: load a model folder, make random weights, build the engine."""
from __future__ import annotations

import json
import os
from typing import Any, Mapping, Optional, Union

import torch

from . import architectures  # noqa: F401  (fills the registry)
from .config.registry import ConfigError, architecture_for
from .engine.engine import Engine
from .weights.loader import load_weights
from .weights.random_init import random_device_weights, write_model_folder

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, torch.bfloat16: torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32, torch.float32: torch.float32,
}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ConfigError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


def read_config(folder: str) -> dict:
    """The configuration keys of a model: config.json of a folder, or the metadata of a .gguf file."""
    if os.path.isfile(folder) and folder.endswith(".gguf"):
        from .weights.gguf import open_gguf
        return open_gguf(folder).config()
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and model.safetensors")
    with open(path) as f:
        return json.load(f)


def _typed(config):
    """(architecture, typed configuration) from a dict of config.json keys."""
    arch = architecture_for(config)
    return arch, arch.config_cls.from_dict(config)


def load(folder: str, dtype="bfloat16", device: Union[str, torch.device] = "cuda:0", *,
         max_tokens: int = 8192, max_slots: Optional[int] = None, max_step_tokens: int = 8192) -> Engine:
    """Engine for the model in ``folder`` (config.json + *.safetensors) or in a ``.gguf`` file (any shard of a sharded one); the
    model class is chosen by the configuration.  ``dtype`` "bfloat16" is the serving path, "float32" the true 32-bit path."""
    dt = parse_dtype(dtype)
    dev = torch.device(device)
    arch, meta = _typed(read_config(folder))
    rules = arch.tensor_plan(meta)
    weights = load_weights(folder, rules, dt, dev)
    return Engine(arch.build_spec(meta), weights, dt, dev, max_tokens=max_tokens, max_slots=max_slots,
                  max_step_tokens=max_step_tokens)


def random_model(config: Mapping[str, Any], seed: int = 0, dtype="bfloat16",
                 device: Union[str, torch.device] = "cuda:0", *, max_tokens: int = 8192,
                 max_slots: Optional[int] = None, max_step_tokens: int = 8192, std: float = 0.02) -> Engine:
    """Engine with random weights drawn on the device (no files)."""
    dt = parse_dtype(dtype)
    dev = torch.device(device)
    arch, meta = _typed(config)
    weights = random_device_weights(arch.tensor_plan(meta), seed, dt, dev, std)
    return Engine(arch.build_spec(meta), weights, dt, dev, max_tokens=max_tokens, max_slots=max_slots,
                  max_step_tokens=max_step_tokens)


def write_random_model(folder: str, config: Mapping[str, Any], seed: int = 0, dtype="bfloat16",
                       std: float = 0.02) -> str:
    """Write config.json and model.safetensors with random weights (matrices in ``dtype``, norm
    weights float32 and equal to one)."""
    arch, meta = _typed(config)
    cfg = meta.to_dict() if hasattr(meta, "to_dict") else dict(config)
    return write_model_folder(folder, cfg, arch.tensor_plan(meta), seed, parse_dtype(dtype), std)
