"""Host-side bookkeeping of the cache: which pages and which sequence slots are free.

Pure Python, no device memory: the storage itself is in ``storage.py``.  Every misuse
(freeing twice, freeing what was never handed out, asking for more than there is) raises
``CacheError`` and changes nothing.
"""
from __future__ import annotations


class CacheError(RuntimeError):
    """The cache cannot do what was asked (out of pages or slots, or a misuse)."""


class FreeList:
    """Integers 0..n-1 handed out lowest-first and taken back exactly once."""

    def __init__(self, n: int, what: str):
        if n <= 0:
            raise CacheError(f"a cache needs at least one {what}")
        self.n, self.what = int(n), what
        self._free = list(range(self.n - 1, -1, -1))     # pop() yields the lowest id
        self._held = [False] * self.n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def take(self, count: int = 1) -> list[int]:
        if count < 0:
            raise CacheError(f"cannot take {count} {self.what}s")
        if count > len(self._free):
            raise CacheError(f"out of {self.what}s: {count} wanted, {len(self._free)} free "
                             f"of {self.n}")
        out = [self._free.pop() for _ in range(count)]
        for i in out:
            self._held[i] = True
        return out

    def give_back(self, ids) -> None:
        ids = list(ids)
        seen = set()
        for i in ids:
            if not (0 <= i < self.n):
                raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
            if not self._held[i] or i in seen:
                raise CacheError(f"{self.what} {i} freed twice or never handed out")
            seen.add(i)
        for i in ids:
            self._held[i] = False
        # keep lowest-first order so that reuse is deterministic
        self._free.extend(ids)
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]


class Sequence:
    """What a live sequence holds: its slot, its pages in order and its length."""
    __slots__ = ("slot", "pages", "length")

    def __init__(self, slot: int):
        self.slot = slot
        self.pages: list[int] = []
        self.length = 0


class SlotTable:
    """Sequence slots and token pages.  A slot is the index of a sequence's fixed-size
    state; pages (``page_size`` tokens each) hold its keys and values."""

    def __init__(self, n_slots: int, n_pages: int, page_size: int):
        if page_size <= 0:
            raise CacheError("page_size must be positive")
        self.page_size = int(page_size)
        self.slots = FreeList(n_slots, "slot")
        self.pages = FreeList(n_pages, "page")
        self.live: dict[int, Sequence] = {}

    def open(self) -> Sequence:
        (slot,) = self.slots.take(1)
        seq = Sequence(slot)
        self.live[slot] = seq
        return seq

    def pages_needed(self, seq: Sequence, new_length: int) -> int:
        want = -(-int(new_length) // self.page_size)
        return max(0, want - len(seq.pages))

    def reserve(self, seq: Sequence, new_length: int) -> list[int]:
        """Makes sure ``seq`` has pages for ``new_length`` tokens; returns the new pages."""
        self._check_live(seq)
        fresh = self.pages.take(self.pages_needed(seq, new_length))
        seq.pages.extend(fresh)
        return fresh

    def close(self, seq: Sequence) -> None:
        self._check_live(seq)
        self.pages.give_back(seq.pages)
        self.slots.give_back([seq.slot])
        del self.live[seq.slot]
        seq.pages = []
        seq.length = 0
        seq.slot = -1

    def _check_live(self, seq: Sequence) -> None:
        if seq.slot < 0 or self.live.get(seq.slot) is not seq:
            raise CacheError("sequence is not live (closed already, or of another cache)")
