"""The one registry from an architecture's name to its model.

config.json's `architectures` list is matched against the registered names, first
match wins, as the reference does (src/wllm/models/registry.py:41-53).  An entry
holds the architecture's configuration class and the function that turns such a
configuration into a `ModelPlan` (the parts of every layer and the order in which
layers run); the engine builds the same `ComposedModel` from any plan.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .base import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    make_plan: Callable  # (config) -> ModelPlan


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type):
    """Decorator for a plan function: @register_architecture("XForCausalLM", XConfig)."""
    def wrap(make_plan: Callable):
        ARCHITECTURES[name] = Architecture(name, config_class, make_plan)
        return make_plan
    return wrap


def resolve_architecture(architectures) -> Architecture:
    _load_builtin()
    names = architectures if isinstance(architectures, (list, tuple)) else [architectures]
    for name in names:
        if name in ARCHITECTURES:
            return ARCHITECTURES[name]
    raise ConfigError(f"unsupported architecture(s) {list(names)!r}; this engine implements: "
                      f"{', '.join(sorted(ARCHITECTURES))}")


def config_from_folder(folder: str):
    """(architecture entry, typed configuration) of a model folder."""
    raw = read_config_json(folder)
    arch = resolve_architecture(raw.get("architectures") or [])
    return arch, arch.config_class.from_dict(raw, where=f"{folder}/config.json")


def _load_builtin() -> None:
    from .. import models  # noqa: F401  (registers the built-in architectures)
