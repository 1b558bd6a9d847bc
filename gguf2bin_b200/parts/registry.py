"""Registries of the part families.  A part is chosen by the ``kind`` of its spec; a new
kind is added with one ``register_*`` call, from anywhere (a test can add a toy part
without touching this package)."""
from __future__ import annotations

from typing import Callable

from ..config.specs import ConfigError, PartSpec

_FAMILIES: dict[str, dict[str, Callable]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {},
    "embedding": {}, "head": {},
}


def _register(family: str, kind: str, cls) -> None:
    _FAMILIES[family][kind] = cls


def _lookup(family: str, spec: PartSpec):
    try:
        return _FAMILIES[family][spec.kind]
    except KeyError:
        raise ConfigError(f"no {family} of kind {spec.kind!r} is registered; registered: "
                          + ", ".join(sorted(_FAMILIES[family]))) from None


def register_norm(kind, cls): _register("norm", kind, cls)
def register_position(kind, cls): _register("position", kind, cls)
def register_mixer(kind, cls): _register("mixer", kind, cls)
def register_feed_forward(kind, cls): _register("feed_forward", kind, cls)
def register_block(kind, cls): _register("block", kind, cls)
def register_embedding(kind, cls): _register("embedding", kind, cls)
def register_head(kind, cls): _register("head", kind, cls)


def norm_class(spec): return _lookup("norm", spec)
def position_class(spec): return _lookup("position", spec)
def mixer_class(spec): return _lookup("mixer", spec)
def feed_forward_class(spec): return _lookup("feed_forward", spec)
def block_class(spec): return _lookup("block", spec)
def embedding_class(spec): return _lookup("embedding", spec)
def head_class(spec): return _lookup("head", spec)


def registered(family: str) -> list[str]:
    return sorted(_FAMILIES[family])
