"""One registry from an architecture's name (``architectures[0]`` of config.json)
to the reader that turns config.json into a ``ModelSpec``."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Callable, Mapping

from .specs import ConfigError, ModelSpec

_ARCHITECTURES: dict[str, Callable[[Mapping[str, Any]], ModelSpec]] = {}


def register_architecture(name: str, reader: Callable[[Mapping[str, Any]], ModelSpec]) -> None:
    """``reader(config_dict) -> ModelSpec``.  Registering a name twice replaces it."""
    _ARCHITECTURES[name] = reader


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def model_spec_from_dict(d: Mapping[str, Any]) -> ModelSpec:
    archs = d.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json: 'architectures' is missing or empty; registered: "
                          + ", ".join(registered_architectures()))
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"config.json: architecture {name!r} is not registered; registered: "
                          + ", ".join(registered_architectures()))
    return _ARCHITECTURES[name](d)


def read_config_json(folder) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no such file")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def model_spec_from_folder(folder) -> ModelSpec:
    return model_spec_from_dict(read_config_json(folder))
