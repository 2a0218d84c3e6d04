"""One registry from an architecture's name to its configuration class and its model description.

The reference has no registry, only a ``model_type`` check (src/cloud_engine/model.py:61-63).
Here ``config.json``'s ``architectures[0]`` (or, when that key is absent, its
``model_type``) selects an entry; an entry is a function from the raw config.json
dictionary to a typed configuration and a function from that configuration to a
``ModelSpec``.  The engine, the loader, the random-weights writer and the replay
program all resolve a model folder through ``resolve_model``.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .model_config import ConfigError, read_config_json
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    parse_config: Callable[[dict[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(
    name: str,
    model_type: str,
    parse_config: Callable[[dict[str, Any]], Any],
    build_spec: Callable[[Any], ModelSpec],
    *,
    replace: bool = False,
) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, model_type, parse_config, build_spec)


def registered_architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_for(raw: dict[str, Any]) -> Architecture:
    names = raw.get("architectures")
    if names:
        name = names[0]
        if name not in _ARCHITECTURES:
            raise ConfigError(
                f"config.json: architecture {name!r} is not registered "
                f"(known: {', '.join(registered_architectures()) or 'none'})"
            )
        return _ARCHITECTURES[name]
    model_type = raw.get("model_type")
    for arch in _ARCHITECTURES.values():
        if arch.model_type == model_type:
            return arch
    raise ConfigError(
        f"config.json: neither 'architectures' nor a known 'model_type' ({model_type!r}) "
        f"selects a model (known: {', '.join(registered_architectures()) or 'none'})"
    )


def resolve_config(raw: dict[str, Any]) -> tuple[Architecture, Any, ModelSpec]:
    """Raw config.json dictionary -> (architecture entry, typed configuration, model description)."""
    arch = architecture_for(raw)
    config = arch.parse_config(raw)
    spec = arch.build_spec(config)
    spec.validate()
    return arch, config, spec


def resolve_model(model_dir: str | Path) -> tuple[Architecture, Any, ModelSpec]:
    return resolve_config(read_config_json(model_dir))
