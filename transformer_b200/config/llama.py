"""Typed configuration of the Llama decoder with an optional mixture-of-experts feed-forward.

Field names and meanings are the reference's ``LlamaMeta`` (models/llama/common/src/lib.rs:19-40);
defaults are the ones its GGUF reader applies (models/llama/common/src/storage.rs:36-60):
``nkvh`` defaults to ``nh``, ``dh`` to ``d / nh``, ``nexp``/``nexp_use`` to 0 (dense feed-forward),
``epsilon`` to 1e-5 and ``theta`` to 1e4.  Every size comes from the file; none stands in code.

Two spellings of every key are accepted: the GGUF metadata key with the ``llama.`` prefix, as the
reference reads it, and the conventional ``config.json`` key.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Mapping

from .registry import ConfigError

# field -> (accepted keys, required, caster)
_KEYS = {
    "nblk": (("num_hidden_layers", "llama.block_count", "nblk"), True, int),
    "d": (("hidden_size", "llama.embedding_length", "d"), True, int),
    "nh": (("num_attention_heads", "llama.attention.head_count", "nh"), True, int),
    "nkvh": (("num_key_value_heads", "llama.attention.head_count_kv", "nkvh"), False, int),
    "dh": (("head_dim", "llama.rope.dimension_count", "dh"), False, int),
    "di": (("intermediate_size", "moe_intermediate_size", "llama.feed_forward_length", "di"), True, int),
    "nexp": (("num_local_experts", "num_experts", "llama.expert_count", "nexp"), False, int),
    "nexp_use": (("num_experts_per_tok", "num_selected_experts", "llama.expert_used_count", "nexp_use"), False, int),
    "nctx": (("max_position_embeddings", "llama.context_length", "nctx"), True, int),
    "nvoc": (("vocab_size", "llama.vocab_size", "nvoc"), True, int),
    "epsilon": (("rms_norm_eps", "llama.attention.layer_norm_rms_epsilon", "epsilon"), False, float),
    "theta": (("rope_theta", "llama.rope.freq_base", "theta"), False, float),
    "tied": (("tie_word_embeddings", "tied"), False, bool),
    "rope_pairing": (("rope_pairing",), False, str),
    "eos": (("eos_token_id", "tokenizer.ggml.eos_token_id"), False, None),
}


@dataclass(frozen=True)
class LlamaMeta:
    nblk: int          # layers
    d: int             # width of the residual stream
    nh: int            # query heads
    nkvh: int          # key/value heads (groups)
    dh: int            # head size
    di: int            # feed-forward width (of one expert when nexp > 0)
    nexp: int          # experts; 0 means a dense feed-forward (lib.rs:74-77)
    nexp_use: int      # experts used per token
    nctx: int          # longest context
    nvoc: int          # vocabulary
    epsilon: float     # RMSNorm epsilon
    theta: float       # RoPE base
    tied: bool = False           # lm_head shares token_embd (storage.rs:84)
    rope_pairing: str = "adjacent"   # "adjacent": (x[2i], x[2i+1]); "half": (x[i], x[i+dh/2])
    eos: tuple = ()              # stop tokens the file declares

    @property
    def is_moe(self) -> bool:
        return self.nexp > 0

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "LlamaMeta":
        got = {}
        missing = []
        for field, (keys, required, cast) in _KEYS.items():
            for k in keys:
                if k in cfg and cfg[k] is not None:
                    v = cfg[k]
                    if cast in (int, float):
                        if isinstance(v, bool) or not isinstance(v, (int, float)):
                            raise ConfigError(f"config key {k!r} must be a number, got {v!r}")
                        if cast is int and int(v) != v:
                            raise ConfigError(f"config key {k!r} must be an integer, got {v!r}")
                        v = cast(v)
                    elif cast is bool:
                        if not isinstance(v, bool):
                            raise ConfigError(f"config key {k!r} must be true or false, got {v!r}")
                    elif cast is str:
                        if not isinstance(v, str):
                            raise ConfigError(f"config key {k!r} must be a string, got {v!r}")
                    got[field] = v
                    break
            else:
                if required:
                    missing.append(" | ".join(keys))
        if missing:
            raise ConfigError("config.json lacks required keys: " + "; ".join(missing))
        if cfg.get("attention_bias") or cfg.get("attn_qkv_bias"):
            raise ConfigError("q/k/v biases are not part of this architecture (storage.rs:45)")
        if cfg.get("sliding_window"):
            raise ConfigError("a sliding window is not part of this architecture")
        got.setdefault("nkvh", got["nh"])
        if "dh" not in got:
            if got["d"] % got["nh"]:
                raise ConfigError(f"hidden_size {got['d']} is not a multiple of the {got['nh']} heads and no head_dim is given")
            got["dh"] = got["d"] // got["nh"]
        got.setdefault("nexp", 0)
        got.setdefault("nexp_use", 0)
        got.setdefault("epsilon", 1e-5)
        got.setdefault("theta", 1e4)
        got.setdefault("tied", False)
        got.setdefault("rope_pairing", "adjacent")
        eos = got.pop("eos", ())
        if isinstance(eos, bool) or not isinstance(eos, (int, list, tuple)):
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        eos = (eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)
        meta = cls(eos=eos, **got)
        meta.validate()
        return meta

    @classmethod
    def from_folder(cls, folder: str) -> "LlamaMeta":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def validate(self) -> None:
        for name in ("nblk", "d", "nh", "nkvh", "dh", "di", "nctx", "nvoc"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.nh % self.nkvh:
            raise ConfigError(f"{self.nh} query heads cannot be shared by {self.nkvh} key/value heads")
        if self.dh % 2:
            raise ConfigError(f"head size {self.dh} must be even for rotary pairs")
        if self.nexp < 0 or self.nexp_use < 0:
            raise ConfigError("expert counts must not be negative")
        if self.nexp > 0 and not (0 < self.nexp_use <= self.nexp):
            raise ConfigError(f"experts per token {self.nexp_use} must lie in 1..{self.nexp}")
        if self.nexp == 0 and self.nexp_use != 0:
            raise ConfigError("experts per token given without experts")
        if not (self.epsilon > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.epsilon}")
        if not (self.theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.theta}")
        if self.rope_pairing not in ("adjacent", "half"):
            raise ConfigError(f"rope_pairing must be 'adjacent' or 'half', got {self.rope_pairing!r}")
        for e in self.eos:
            if not (0 <= e < self.nvoc):
                raise ConfigError(f"eos token {e} lies outside the vocabulary of {self.nvoc}")

    # ---- serialisation ------------------------------------------------------------------
    def to_dict(self) -> dict:
        """The keys this class reads back, in the conventional config.json spelling."""
        out = {
            "model_type": "llama",
            "architectures": ["LlamaMoe" if self.is_moe else "Llama"],
            "num_hidden_layers": self.nblk,
            "hidden_size": self.d,
            "num_attention_heads": self.nh,
            "num_key_value_heads": self.nkvh,
            "head_dim": self.dh,
            "intermediate_size": self.di,
            "num_local_experts": self.nexp,
            "num_experts_per_tok": self.nexp_use,
            "max_position_embeddings": self.nctx,
            "vocab_size": self.nvoc,
            "rms_norm_eps": self.epsilon,
            "rope_theta": self.theta,
            "tie_word_embeddings": self.tied,
            "rope_pairing": self.rope_pairing,
        }
        if self.eos:
            out["eos_token_id"] = list(self.eos)
        return out

    def describe(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}
