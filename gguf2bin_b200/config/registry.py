"""One registry from an architecture's name (``architectures[0]`` of config.json)
to the reader that turns config.json into a ``ModelSpec``."""
from __future__ import annotations

import dataclasses
import importlib
import json
import os
from pathlib import Path
from typing import Any, Callable, Mapping

from .specs import ConfigError, ModelSpec

_ARCHITECTURES: dict[str, Callable[[Mapping[str, Any]], ModelSpec]] = {}


def register_architecture(name: str, reader: Callable[[Mapping[str, Any]], ModelSpec]) -> None:
    """``reader(config_dict) -> ModelSpec``.  Registering a name twice replaces it."""
    _ARCHITECTURES[name] = reader


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


_plugins_loaded = False


def load_plugins() -> None:
    """Imports the modules named in ``GGUF2BIN_B200_PLUGINS`` (comma-separated, importable from
    ``sys.path``), once.  A module adds an architecture, or kinds of parts, by calling the
    ``register_*`` functions when it is imported; that is how a model that this package does not
    know reaches every entry point (the Python API, the command line, ``bin/trace_run``) without a
    change to the package's files."""
    global _plugins_loaded
    if _plugins_loaded:
        return
    _plugins_loaded = True
    for name in os.environ.get("GGUF2BIN_B200_PLUGINS", "").split(","):
        name = name.strip()
        if not name:
            continue
        try:
            importlib.import_module(name)
        except ImportError as e:
            raise ConfigError(f"GGUF2BIN_B200_PLUGINS: cannot import {name!r}: {e}") from None


def model_spec_from_dict(d: Mapping[str, Any]) -> ModelSpec:
    load_plugins()
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


def _id_list(v, where: str) -> tuple:
    if v is None:
        return ()
    items = v if isinstance(v, (list, tuple)) else [v]
    for e in items:
        if isinstance(e, bool) or not isinstance(e, int):
            raise ConfigError(f"{where}: eos_token_id must be an integer or a list of integers, got {v!r}")
    return tuple(int(e) for e in items)


def read_generation_stop_ids(folder) -> tuple:
    """``eos_token_id`` of the folder's generation_config.json (one id or a list); () when
    the file is absent.  The reference ends a reply at the tokenizer's eos or at
    ``<|im_end|>`` (src/main.c:387-389 of AnonymoDGH/gguf2bin); without a tokenizer the ids
    come from the two configuration files that carry them."""
    path = Path(folder) / "generation_config.json"
    if not path.is_file():
        return ()
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return _id_list(d.get("eos_token_id"), str(path))


def model_spec_from_folder(folder) -> ModelSpec:
    """The folder's config.json through the registry; stop ids are those of config.json
    and of generation_config.json together, in that order."""
    spec = model_spec_from_dict(read_config_json(folder))
    extra = [t for t in read_generation_stop_ids(folder) if t not in spec.stop_token_ids]
    if extra:
        spec = dataclasses.replace(spec, stop_token_ids=tuple(spec.stop_token_ids) + tuple(extra))
    return spec
