"""The cache: sequence slots, token pages, per-slot fixed-size state, and storage per
group of layers with equal needs."""
from .pool import CacheError, FreeList, Sequence, SlotTable
from .storage import (PAGE_SIZE, SEQ_STATE_WORDS, SS_DRAWS, SS_RECENT_TOTAL, SS_RING, SS_RING_WORDS, SS_SEED_HI,
                      SS_SEED_LO, SS_STREAM,
                      Cache, KVNeed, KVView, StateNeed, StateView)

__all__ = ["CacheError", "FreeList", "Sequence", "SlotTable", "PAGE_SIZE", "SEQ_STATE_WORDS",
           "SS_DRAWS", "SS_RECENT_TOTAL", "SS_RING", "SS_RING_WORDS", "SS_SEED_HI", "SS_SEED_LO", "SS_STREAM", "Cache", "KVNeed", "KVView",
           "StateNeed", "StateView"]
