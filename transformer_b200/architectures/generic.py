"""A tensor plan derived from a ModelSpec alone, for architectures that have no file format of
their own (experiments, tests): every parameter a part declares becomes one file tensor named

    embedding.table, head.weight (absent when the head is tied), final_norm.<param>,
    layers.<i>.<mixer_norm | mixer | feed_forward_norm | feed_forward>.<param>
"""
from __future__ import annotations

from typing import List

import torch

from ..parts.base import NORMS
from ..parts.block import Layer
from ..parts.spec import ModelSpec
from ..weights.plan import TensorRule, single


def plan_from_spec(spec: ModelSpec) -> List[TensorRule]:
    cpu = torch.device("cpu")
    V, d = spec.vocab, spec.width
    rules = [TensorRule(("embedding", "table"), (V, d), "matrix", (single("embedding.table", (V, d)),))]
    for i, ls in enumerate(spec.layers):
        layer = Layer(ls, torch.bfloat16, cpu)
        for pname, part in layer.parts().items():
            for name, decl in part.parameters().items():
                rules.append(TensorRule(("layers", i, pname, name), tuple(decl.shape), decl.role,
                                        (single(f"layers.{i}.{pname}.{name}", decl.shape),), init=decl.init))
    fn = NORMS.build(spec.final_norm, torch.bfloat16, cpu)
    for name, decl in fn.parameters().items():
        rules.append(TensorRule(("final_norm", name), tuple(decl.shape), decl.role,
                                (single(f"final_norm.{name}", decl.shape),), init=decl.init))
    tied = bool(spec.head.get().get("tied", False))
    rules.append(TensorRule(("head", "weight"), (V, d), "matrix", (single("head.weight", (V, d)),),
                            shared_with=("embedding", "table") if tied else None))
    return rules
