"""One registry from the architecture name in config.json to the model recipe."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from ..config.errors import ConfigError, UnknownArchitectureError
from ..parts.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    """`config_from_dict` reads config.json's keys into a typed configuration (any object:
    only `build_spec` looks inside it); `build_spec` turns that configuration into a
    `ModelSpec`, the description of parts that everything else works from: loader, cache,
    step, generation, command line and replay read sizes, stop tokens and the longest
    sequence from the `ModelSpec` alone."""
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    ARCHITECTURES[arch.name] = arch
    return arch


def architecture_for(config_dict: Mapping[str, Any]) -> Architecture:
    """Look the model up by config.json["architectures"][0]."""
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names; "
                          f"known architectures: {sorted(ARCHITECTURES)}")
    name = archs[0]
    if name not in ARCHITECTURES:
        raise UnknownArchitectureError(
            f"config.json names architecture '{name}', which is not registered; "
            f"known architectures: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[name]
