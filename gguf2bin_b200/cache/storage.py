"""Device storage of the cache.

Every execution of a layer (a position of the model's schedule) says what it needs
through a ``KVNeed`` or ``StateNeed``; positions with equal needs share one group, and
every group has storage of its own:

* ``KVNeed``: keys and values of every position (``window == 0``) or of a window of
  them.  Storage ``[layers, pages, 2 (K,V), kv_heads, page_size, head_dim]``: one
  (page, kv head) panel of keys is contiguous, so a kernel streams it with full-width
  loads.  Page numbers are shared by all groups: page ``p`` of a sequence covers the same
  token range everywhere.
* ``StateNeed``: a fixed-size state per sequence (for mixers that carry a state instead
  of keys).  Storage ``[layers, slots, *shape]``, cleared when a slot is opened.

Beside the groups there is one fixed-size record per slot, ``seq_state``
(``[slots, SEQ_STATE_WORDS]`` int32): the sampler's key and draw counter live there, so
a sequence's random stream does not depend on the batch it is in, and so do the sequence's
most recent tokens (a ring of ``SS_RING_WORDS`` ids and the count of tokens written to it),
which the repeat penalty reads on the device.

Every storage has one page and one slot more than the table hands out (``spare_page``,
``spare_slot``): a step that runs more rows than it has sequences, to keep a shape it has
launches for, points the extra rows there; what they write is never read by a sequence.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence as Seq

import torch

from .pool import CacheError, Sequence, SlotTable

PAGE_SIZE = 64
# word indices of the per-slot record (the same numbers as in csrc/sampling.cu)
SS_SEED_LO, SS_SEED_HI, SS_STREAM, SS_DRAWS, SS_RECENT_TOTAL = 0, 1, 2, 3, 4
SS_RING, SS_RING_WORDS = 8, 72           # ring of recent token ids: the last 64 are used, 8 spare for a step taken back
SEQ_STATE_WORDS = SS_RING + SS_RING_WORDS


@dataclass(frozen=True)
class KVNeed:
    n_kv_heads: int
    head_dim: int
    window: int = 0          # 0: every position is kept

    @property
    def group_key(self):
        return ("kv", self.n_kv_heads, self.head_dim, "window" if self.window else "full")


@dataclass(frozen=True)
class StateNeed:
    shape: tuple
    dtype: torch.dtype = torch.float32

    @property
    def group_key(self):
        return ("state", tuple(self.shape), self.dtype)


@dataclass
class KVView:
    """What an attention mixer gets for one layer: the layer's K/V pages."""
    pages: torch.Tensor       # [n_pages, 2, n_kv_heads, page_size, head_dim]
    page_size: int


@dataclass
class StateView:
    states: torch.Tensor      # [n_slots, *shape]


class Cache:
    """Slots, pages, per-slot state and the groups' storage for one model."""

    def __init__(self, needs: Seq[Optional[object]], max_tokens: int, dtype: torch.dtype, device,
                 max_seqs: Optional[int] = None, page_size: int = PAGE_SIZE):
        """``needs[i]`` is the need of schedule position ``i`` (None: it stores nothing, or
        uses another position's storage).  ``max_tokens`` is the most tokens live sequences
        hold together, each sequence rounded up to whole pages."""
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        self.page_size = int(page_size)
        n_pages = -(-int(max_tokens) // self.page_size)
        n_slots = int(max_seqs) if max_seqs else min(n_pages, 512)
        self.table = SlotTable(n_slots, n_pages, self.page_size)
        self.dtype, self.device = dtype, torch.device(device)
        self.n_pages, self.n_slots = n_pages, n_slots
        self.spare_page, self.spare_slot = n_pages, n_slots          # beyond what the table hands out
        self.groups: dict[tuple, dict] = {}
        self._layer_group: dict[int, tuple] = {}
        for layer, need in enumerate(needs):
            if need is None:
                continue
            g = self.groups.setdefault(need.group_key, {"need": need, "layers": []})
            g["layers"].append(layer)
            self._layer_group[layer] = (need.group_key, len(g["layers"]) - 1)
        for key, g in self.groups.items():
            need, nl = g["need"], len(g["layers"])
            if isinstance(need, KVNeed):
                g["storage"] = torch.zeros(
                    (nl, n_pages + 1, 2, need.n_kv_heads, self.page_size, need.head_dim),
                    dtype=dtype, device=self.device)
            else:
                g["storage"] = torch.zeros((nl, n_slots + 1) + tuple(need.shape), dtype=need.dtype,
                                           device=self.device)
        self.seq_state = torch.zeros((n_slots + 1, SEQ_STATE_WORDS), dtype=torch.int32,
                                     device=self.device)
        self._views: dict = {}

    # ---- sequences ---------------------------------------------------------
    def open_sequence(self) -> Sequence:
        seq = self.table.open()
        for g in self.groups.values():
            if isinstance(g["need"], StateNeed):
                g["storage"][:, seq.slot].zero_()
        self.seq_state[seq.slot].zero_()
        return seq

    def close_sequence(self, seq: Sequence) -> None:
        self.table.close(seq)

    def reserve(self, seq: Sequence, new_length: int) -> list[int]:
        return self.table.reserve(seq, new_length)

    # ---- views -------------------------------------------------------------
    def view(self, layer: int):
        """The layer's part of its group's storage (made once: the storage never moves)."""
        v = self._views.get(layer, self)
        if v is self:
            if layer not in self._layer_group:
                v = None
            else:
                key, idx = self._layer_group[layer]
                g = self.groups[key]
                v = (KVView(g["storage"][idx], self.page_size) if isinstance(g["need"], KVNeed)
                     else StateView(g["storage"][idx]))
            self._views[layer] = v
        return v

    def bytes(self) -> int:
        return sum(g["storage"].numel() * g["storage"].element_size()
                   for g in self.groups.values())

    def describe(self) -> str:
        parts = [f"{len(g['layers'])} layers x {k[0]}{k[1:]}" for k, g in self.groups.items()]
        return (f"cache: {self.n_pages} pages of {self.page_size} tokens, {self.n_slots} slots, "
                f"{self.bytes() / 2**20:.1f} MiB, {self.dtype}; groups: " + "; ".join(parts))
