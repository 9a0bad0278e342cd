"""One registry from an architecture's name to how its model is made.

An entry turns the architecture's config.json into a typed configuration and that
into a `ModelSpec` (which parts, which sizes, which tensor names, which order).
arhaamatiq/stride has no such registry: its loader never looks at `architectures`
(src/model.cpp:15-52); it is here so that another architecture is one more entry.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .llama import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable      # dict (config.json) -> typed configuration
    model_spec: Callable        # typed configuration -> ModelSpec


_ARCHITECTURES: dict = {}


def register_architecture(arch: Architecture, *aliases: str) -> None:
    for key in (arch.name, *aliases):
        _ARCHITECTURES[key] = arch


def registered_architectures() -> list:
    return sorted(_ARCHITECTURES)


def resolve_architecture(config: dict) -> Architecture:
    """Chosen by config.json's `architectures[0]`, else by `model_type`."""
    names = list(config.get("architectures") or [])
    if config.get("model_type"):
        names.append(config["model_type"])
    if not names:
        raise ConfigError("config.json names no architecture (keys 'architectures' or 'model_type'); "
                          f"registered: {', '.join(registered_architectures())}")
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise ConfigError(f"architecture {names[0]!r} is not registered; registered: {', '.join(registered_architectures())}")
