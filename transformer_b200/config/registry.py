"""One registry from an architecture's name to everything that builds its model.

An :class:`Architecture` bundles four things and nothing else knows which model it is in:

* ``config_cls.from_dict``   -- typed configuration from the keys of ``config.json``
* ``build_spec(config)``     -- the model as data: layers made of parts, and the order they run in
* ``tensor_plan(config)``    -- which file tensor (by name) fills which parameter of which part
* ``names``                  -- the strings ``config.json`` may carry in ``model_type`` /
                                ``architectures`` / ``general.architecture``

The reference has no such table: each model is a crate of its own and the only dispatch on the
architecture string is ``arch == "qwen2"`` (models/llama/common/src/storage.rs:31,45).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Mapping


class ConfigError(ValueError):
    """A configuration key is missing, has the wrong type, or the sizes contradict each other."""


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any
    build_spec: Callable[[Any], Any]
    tensor_plan: Callable[[Any], Any]
    names: tuple = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    keys = {arch.name, *arch.names}
    for key in keys:
        k = key.lower()
        if k in _ARCHITECTURES and _ARCHITECTURES[k] is not arch and not replace:
            raise ConfigError(f"architecture name {key!r} is already registered")
    for key in keys:
        _ARCHITECTURES[key.lower()] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _ARCHITECTURES.get(name.lower())
    if arch is None:
        return
    for key in [k for k, v in _ARCHITECTURES.items() if v is arch]:
        del _ARCHITECTURES[key]


def registered_architectures() -> Iterable[str]:
    return sorted({a.name for a in _ARCHITECTURES.values()})


def architecture_names_in(config: Mapping[str, Any]) -> list:
    """Every string of a config.json that may name the architecture, most specific first."""
    found = []
    for key in ("general.architecture", "model_type"):
        v = config.get(key)
        if isinstance(v, str):
            found.append(v)
    v = config.get("architectures")
    if isinstance(v, (list, tuple)):
        found.extend(x for x in v if isinstance(x, str))
    elif isinstance(v, str):
        found.append(v)
    return found


def architecture_for(config: Mapping[str, Any]) -> Architecture:
    names = architecture_names_in(config)
    if not names:
        raise ConfigError(
            "config.json names no architecture: expected one of the keys "
            "'model_type', 'architectures' or 'general.architecture'"
        )
    for n in names:
        arch = _ARCHITECTURES.get(n.lower())
        if arch is not None:
            return arch
    raise ConfigError(
        f"unknown architecture {names!r}; registered: {list(registered_architectures())}"
    )
