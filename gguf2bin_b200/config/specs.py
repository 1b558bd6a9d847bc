"""Typed descriptions of a model: which parts each layer is made of, and in which
order layers run.

A ``ModelSpec`` is pure data.  It is what an architecture's configuration reader
produces from ``config.json`` and what the engine builds a model from.  Every size
and constant of a part lives in that part's spec; nothing about the parts is
implied by the architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional


class ConfigError(ValueError):
    """A configuration that cannot be built, with the reason."""


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by ``kind`` (a name in that part family's registry) with its
    parameters.  ``params`` holds only plain values so that specs compare and hash."""
    kind: str
    params: tuple = ()

    @staticmethod
    def make(kind: str, **params: Any) -> "PartSpec":
        return PartSpec(kind, tuple(sorted(params.items())))

    def get(self, key: str, default: Any = None) -> Any:
        for k, v in self.params:
            if k == key:
                return v
        return default

    def __getitem__(self, key: str) -> Any:
        for k, v in self.params:
            if k == key:
                return v
        raise KeyError(f"{self.kind} spec has no parameter {key!r}")

    def as_dict(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward, the norm
    used in the block (``ffn_norm``: another one before the feed-forward, when the two
    places differ), and the tensor-name prefix of the layer in the checkpoint."""
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec
    prefix: str
    ffn_norm: Optional[PartSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  Every execution has cache storage of its own (a layer
    that is named twice runs with the same weights but keeps two caches), unless
    ``cache_of`` names an EARLIER position of the schedule: then this execution uses the
    storage of that one (a layer that reads another layer's keys and values)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: tuple                     # tuple[LayerSpec, ...]
    schedule: tuple                   # tuple[ScheduleEntry, ...]
    embedding: PartSpec               # kind "token_embedding"
    final_norm: PartSpec
    head: PartSpec                    # kind "lm_head" (tied or own matrix)
    stop_token_ids: tuple = ()
    source: Mapping[str, Any] = field(default_factory=dict, compare=False, hash=False)

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0 or self.max_positions <= 0:
            raise ConfigError("hidden_size, vocab_size and max_positions must be positive")
        if self.vocab_size >= 2 ** 31:
            raise ConfigError("vocab_size does not fit a 32-bit token id")
        if not self.layers or not self.schedule:
            raise ConfigError("a model needs at least one layer and one schedule entry")
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < n):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, outside 0..{n - 1}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ConfigError(f"schedule entry {i}: cache_of={e.cache_of} must name an "
                                      "earlier entry of the schedule")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {i}: cache_of={e.cache_of} names an entry "
                                      "that itself borrows its storage")

    def cache_owner(self, position: int) -> int:
        """The schedule position whose storage the execution at ``position`` uses."""
        e = self.schedule[position]
        return position if e.cache_of is None else e.cache_of
