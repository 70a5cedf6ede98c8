"""transformer_b200: a small, whole generation library for one GPU (NVIDIA B200, sm_100a).

    import transformer_b200 as tb
    engine = tb.load("model_dir", dtype="bfloat16")          # or tb.random_model(config, seed)
    out = tb.generate(engine, prompts, max_steps=32)          # token ids in, token ids out
"""
from .api import load, parse_dtype, random_model, read_config, write_random_model
from .config import ConfigError, LlamaMeta, register_architecture
from .engine import Engine, StepError, generate, GenerationResult
from .sampling import SampleArgs, SampleArgsError
from .cache import CacheError
from .csrc.lib import KernelError
from .weights import WeightError

__all__ = ["load", "random_model", "write_random_model", "read_config", "parse_dtype", "Engine", "LlamaMeta", "generate", "GenerationResult", "SampleArgs", "SampleArgsError",
           "ConfigError", "WeightError", "CacheError", "StepError", "KernelError", "register_architecture"]
