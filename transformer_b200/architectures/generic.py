"""A tensor plan derived from a ModelSpec alone, for architectures that have no file format of
their own (experiments, tests): every parameter a part declares becomes one file tensor named

    embedding.<param>, head.<param> (``head.weight`` is absent when the head is tied), final_norm.<param>,
    layers.<i>.<part of the block>.<param>       (pre_norm: mixer_norm | mixer | feed_forward_norm | feed_forward)
"""
from __future__ import annotations

from typing import List

import torch

from ..parts.base import EMBEDDINGS, HEADS, NORMS
from ..parts.block import build_layer
from ..parts.spec import ModelSpec
from ..weights.plan import TensorRule, single


def plan_from_spec(spec: ModelSpec) -> List[TensorRule]:
    cpu = torch.device("cpu")
    rules = []

    def declare(dest, file_prefix, part, tied_to=None):
        for name, decl in part.parameters().items():
            shared = tied_to if (tied_to is not None and name == "weight") else None
            rules.append(TensorRule(dest + (name,), tuple(decl.shape), decl.role,
                                    (single(f"{file_prefix}.{name}", decl.shape),), init=decl.init, shared_with=shared))

    declare(("embedding",), "embedding", EMBEDDINGS.build(spec.embedding, torch.bfloat16, cpu))
    for i, ls in enumerate(spec.layers):
        for pname, part in build_layer(ls, torch.bfloat16, cpu).parts().items():
            declare(("layers", i, pname), f"layers.{i}.{pname}", part)
    declare(("final_norm",), "final_norm", NORMS.build(spec.final_norm, torch.bfloat16, cpu))
    tied = bool(spec.head.get().get("tied", False))
    declare(("head",), "head", HEADS.build(spec.head, torch.bfloat16, cpu),
            tied_to=("embedding", "table") if tied else None)
    return rules
