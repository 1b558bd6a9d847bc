"""The cache's bookkeeping: no slot or page lost, held twice or freed twice; groups of
layers with different needs get storage of their own."""
import random

import pytest
import torch

from gguf2bin_b200.cache import (Cache, CacheError, FreeList, KVNeed, SlotTable, StateNeed)


def test_free_list_hands_out_each_id_once():
    f = FreeList(5, "page")
    got = f.take(3)
    assert got == [0, 1, 2] and f.n_free == 2 and f.n_held == 3
    with pytest.raises(CacheError, match="out of pages"):
        f.take(3)
    assert f.n_free == 2                                  # a refused take changes nothing
    f.give_back([1])
    with pytest.raises(CacheError, match="freed twice"):
        f.give_back([1])
    with pytest.raises(CacheError, match="freed twice"):
        f.give_back([0, 0])
    assert f.is_held(0)                                   # the refused call freed nothing
    with pytest.raises(CacheError, match="does not exist"):
        f.give_back([7])
    assert f.take(1) == [1]                               # lowest free id first


def test_slot_table_random_walk_conserves_everything():
    rng = random.Random(0)
    table = SlotTable(n_slots=6, n_pages=40, page_size=64)
    live = []
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and table.slots.n_free:
            live.append(table.open())
        elif op < 0.7 and live:
            s = rng.choice(live)
            want = s.length + rng.randint(1, 200)
            need = table.pages_needed(s, want)
            if need <= table.pages.n_free:
                fresh = table.reserve(s, want)
                assert len(fresh) == need
                s.length = want
            else:
                with pytest.raises(CacheError):
                    table.reserve(s, want)
        elif live:
            s = live.pop(rng.randrange(len(live)))
            table.close(s)
            with pytest.raises(CacheError, match="not live"):
                table.close(s)
        held_pages = [p for s in live for p in s.pages]
        assert len(held_pages) == len(set(held_pages)) == table.pages.n_held
        assert len({s.slot for s in live}) == len(live) == table.slots.n_held
        assert table.pages.n_held + table.pages.n_free == 40
        for s in live:
            assert len(s.pages) * 64 >= s.length
    for s in live:
        table.close(s)
    assert table.pages.n_free == 40 and table.slots.n_free == 6


def test_freed_slots_and_pages_are_used_again():
    table = SlotTable(2, 4, 64)
    a, b = table.open(), table.open()
    table.reserve(a, 128)
    table.reserve(b, 65)
    with pytest.raises(CacheError, match="out of slots"):
        table.open()
    pages_a, slot_a = list(a.pages), a.slot
    table.close(a)
    c = table.open()
    assert c.slot == slot_a
    assert table.reserve(c, 100) == pages_a


def test_groups_have_storage_of_their_own():
    needs = [KVNeed(2, 16), KVNeed(2, 16, window=8), None, KVNeed(2, 16), StateNeed((5, 3)),
             KVNeed(1, 32)]
    cache = Cache(needs, max_tokens=200, dtype=torch.float32, device="cpu", max_seqs=3)
    assert cache.n_pages == 4 and cache.page_size == 64
    assert len(cache.groups) == 4
    full, win, st, other = cache.view(0), cache.view(1), cache.view(4), cache.view(5)
    assert cache.view(2) is None
    assert tuple(full.pages.shape) == (5, 2, 2, 64, 16) and tuple(other.pages.shape) == (5, 2, 1, 64, 32)   # one spare page
    assert tuple(st.states.shape) == (4, 5, 3)                    # and one spare slot
    assert cache.spare_page == 4 and cache.spare_slot == 3
    ptrs = {v.pages.data_ptr() for v in (full, win, cache.view(3), other)}
    assert len(ptrs) == 4                                  # layers 0 and 3 share a group, not storage
    assert full.pages.untyped_storage().data_ptr() == cache.view(3).pages.untyped_storage().data_ptr()
    assert full.pages.untyped_storage().data_ptr() != win.pages.untyped_storage().data_ptr()
    # opening a slot clears its fixed-size state and its record, not the others'
    st.states.fill_(7.0)
    cache.seq_state.fill_(9)
    s = cache.open_sequence()
    assert st.states[s.slot].abs().sum() == 0 and st.states[1:].min() == 7.0
    assert cache.seq_state[s.slot].abs().sum() == 0 and cache.seq_state[1:].min() == 9
    cache.close_sequence(s)
    with pytest.raises(CacheError):
        cache.close_sequence(s)
    with pytest.raises(CacheError):
        Cache(needs, max_tokens=0, dtype=torch.float32, device="cpu")
