"""One registry from an architecture's name to what builds its model.

The reference maps a GGUF `general.architecture` string to an `Arch` variant
and falls back to Llama for a name it does not know (src/arch.rs:134-142,
src/model.rs:181-189).  A library should not guess: an unknown name is an
error here, and the message lists the names that are known.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .errors import ConfigError
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    """name: the string in config.json's `architectures`.
    parse: config.json (a dict) -> typed configuration.
    describe: typed configuration -> ModelSpec."""

    name: str
    parse: Callable[[Mapping[str, Any]], Any]
    describe: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{arch.name}' is already registered")
    _ARCHITECTURES[arch.name] = arch


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(config_json: Mapping[str, Any]) -> str:
    names = config_json.get("architectures")
    if not isinstance(names, (list, tuple)) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError(f"config.json must name exactly one architecture in 'architectures', got {names!r}")
    return names[0]


def lookup_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture '{name}' (known: {', '.join(known_architectures()) or 'none'})") from None


def parse_config(config_json: Mapping[str, Any]):
    """config.json -> (Architecture, typed configuration)."""
    arch = lookup_architecture(architecture_name(config_json))
    return arch, arch.parse(config_json)


def describe_model(config_json: Mapping[str, Any]) -> ModelSpec:
    arch, cfg = parse_config(config_json)
    spec = arch.describe(cfg)
    spec.validate()
    return spec
