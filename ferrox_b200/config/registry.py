"""The one registry: architecture name -> (typed configuration, model description).

``config.json`` names its architecture in ``architectures[0]``; everything else in
the framework (loader, engine, trace replay, command line) asks this registry for
the model that belongs to that name.  An unknown name fails closed with the list of
known ones, as the reference's capability table does
(crates/ferrox-models/src/capability.rs:603-611, loader.rs:52-58,118-123).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .schema import ConfigError, load_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_json: Callable[[dict], object]  # dict -> typed config (raises ConfigError)
    model_spec: Callable[[object], object]  # typed config -> parts.specs.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_json, model_spec, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_from_json, model_spec)


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_of(obj: dict, where: str = "config.json") -> Architecture:
    archs = obj.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: 'architectures' must be a non-empty list of names")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"{where}: unsupported architecture {name!r}; known: {', '.join(known_architectures())}"
        )
    return _ARCHITECTURES[name]


def resolve(config) -> tuple:
    """``config`` is a model folder, a path to a config.json, or the parsed dict.
    Returns (typed config, ModelSpec)."""
    obj = load_json(config) if isinstance(config, str) else config
    arch = architecture_of(obj)
    typed = arch.config_from_json(obj)
    return typed, arch.model_spec(typed)
