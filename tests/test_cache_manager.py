"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders."""
import random

import pytest
import torch

from torchinferno_b200.cache.manager import CacheError, CacheManager, OutOfPages, PageAllocator
from torchinferno_b200.parts.base import CacheSpec, StateSpec


def manager(num_pages=8, page_size=4, specs=None, states=None, max_requests=4, max_request_tokens=64, tensors=False):
    specs = specs or [CacheSpec(2, 16)] * 2
    return CacheManager(specs, states or [None] * len(specs), page_size=page_size, num_pages=num_pages,
                        max_requests=max_requests, max_request_tokens=max_request_tokens, dtype=torch.float32,
                        device="cpu", allocate_tensors=tensors)


def test_allocator_lowest_first_lifo_reuse_and_double_free():
    a = PageAllocator(4)
    assert [a.alloc() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(OutOfPages):
        a.alloc()
    a.release(2), a.release(0)
    assert a.alloc() == 0 and a.alloc() == 2          # last freed is reused first
    a.release(1)
    with pytest.raises(CacheError, match="twice"):
        a.release(1)
    with pytest.raises(CacheError):
        a.release(9)
    a.retain(3)
    a.release(3)
    assert a.num_free == 1 and a.refcount(3) == 1     # still held by the other holder
    a.release(3)
    assert a.num_free == 2


def test_pages_come_as_tokens_arrive_and_go_back_at_the_end():
    m = manager()
    assert m.open("a") == 0 and m.extend("a", 5) == 0
    assert m.block_table("a") == [0, 1] and m.length("a") == 5 and m.free_pages() == [6]
    assert m.extend("a", 3) == 5 and m.block_table("a") == [0, 1]          # fills the second page
    assert m.extend("a", 1) == 8 and m.block_table("a") == [0, 1, 2]
    m.open("b"), m.extend("b", 4)
    assert m.block_table("b") == [3]
    m.audit()
    m.close("a")
    assert m.free_pages() == [7] and "a" not in m
    m.open("c"), m.extend("c", 9)
    assert m.block_table("c") == [2, 1, 0]                                   # pages of "a" are used again
    m.audit()
    with pytest.raises(CacheError):
        m.close("a")
    with pytest.raises(CacheError):
        m.extend("zzz", 1)
    with pytest.raises(CacheError, match="already open"):
        m.open("b")


def test_out_of_pages_changes_nothing():
    m = manager(num_pages=3)
    m.open("a"), m.extend("a", 8)
    m.open("b")
    assert not m.can_extend("b", 5) and m.can_extend("b", 4)
    with pytest.raises(OutOfPages):
        m.extend("b", 5)
    assert m.length("b") == 0 and m.block_table("b") == [] and m.free_pages() == [1]
    m.extend("b", 4)
    m.audit()


def test_groups_have_pools_of_their_own_and_windows_release_early():
    specs = [CacheSpec(2, 16), CacheSpec(2, 16, window=6), CacheSpec(2, 16), CacheSpec(1, 32, window=6)]
    m = manager(num_pages=6, specs=specs, max_request_tokens=24)
    assert len(m.groups) == 3 and m.groups[0].cache_layers == [0, 2] and m.groups[1].cache_layers == [1]
    assert m.group_of_layer(3) == 2
    m.open("a")
    m.extend("a", 12)
    assert m.free_pages() == [3, 3, 3]
    # next query stands at 12 and reads keys >= 7: the first page (keys 0..3) has passed the window
    assert m.release_behind_window("a") == 2
    assert m.block_table("a", 0) == [0, 1, 2] and m.block_table("a", 1) == [-1, 1, 2] and m.free_pages() == [3, 4, 4]
    m.extend("a", 8)
    m.release_behind_window("a")
    assert m.block_table("a", 1)[:3] == [-1, -1, -1] and m.block_table("a", 0) == [0, 1, 2, 3, 4]
    m.audit()
    m.close("a")
    assert m.free_pages() == [6, 6, 6]
    m.audit()


def test_table_updates_are_queued_once():
    m = manager()
    m.open("a"), m.extend("a", 6)
    (index, value), = m.drain_table_updates()
    stride = m.max_pages_per_request
    assert index == [0 * stride + 0, 0 * stride + 1] and value == [0, 1]
    assert m.drain_table_updates() == [([], [])]
    m.close("a")
    (index, value), = m.drain_table_updates()
    assert value == [-1, -1]


def test_state_slots_are_zeroed_and_reused():
    m = manager(states=[StateSpec((3,)), None], tensors=True)
    slot = m.open("a")
    m.state(0)[slot] += 5
    m.close("a")
    assert m.open("b") == slot and torch.all(m.state(0)[slot] == 0) and m.state(1) is None
    for name in "cde":
        m.open(name)
    with pytest.raises(CacheError, match="slots"):
        m.open("f")
    m.audit()


def test_request_limit():
    m = manager(max_request_tokens=10)
    m.open("a")
    with pytest.raises(CacheError, match="limit"):
        m.extend("a", 11)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_double_a_page(seed):
    rng = random.Random(seed)
    specs = [CacheSpec(2, 16), CacheSpec(2, 16, window=rng.choice([3, 5, 9]))]
    m = manager(num_pages=rng.choice([5, 9, 16]), page_size=rng.choice([1, 3, 4]), specs=specs,
                max_requests=5, max_request_tokens=40)
    live, counter = [], 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and m.free_slots():
            counter += 1
            m.open(counter)
            live.append(counter)
        elif action < 0.75 and live:
            rid = rng.choice(live)
            n = rng.randint(1, 7)
            before = (m.length(rid), m.free_pages(), m.block_table(rid, 0), m.block_table(rid, 1))
            if m.length(rid) + n > 40:
                continue
            try:
                start = m.extend(rid, n)
                assert start == before[0] and m.length(rid) == start + n
                m.release_behind_window(rid)
            except OutOfPages:
                assert before == (m.length(rid), m.free_pages(), m.block_table(rid, 0), m.block_table(rid, 1))
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            m.close(rid)
        m.audit()
        for rid in live:                      # every readable key has a page
            for g, spec in enumerate(s for s in specs):
                table = m.block_table(rid, g)
                lo = max(0, m.length(rid) - spec.window + 1) if spec.window else 0
                for pos in range(lo, m.length(rid)):
                    assert table[pos // m.page_size] >= 0
    for rid in live:
        m.close(rid)
    m.audit()
    assert m.free_pages() == [m.num_pages] * 2


def test_a_slot_reused_between_two_steps_queues_each_table_entry_once():
    m = manager()
    m.open("a"), m.extend("a", 6)
    m.drain_table_updates()
    m.close("a")
    m.open("b"), m.extend("b", 3)                     # same slot, first entry set again
    (index, value), = m.drain_table_updates()
    assert sorted(index) == [0, 1] and len(set(index)) == len(index)
    assert dict(zip(index, value)) == {0: m.block_table("b")[0], 1: -1}


def test_a_request_record_is_written_whole_when_the_slot_is_opened():
    """Every word of the slot's record is queued at open (nothing of the last holder stays), later changes replace
    queued ones word by word, and the queue empties when it is drained."""
    import struct
    from torchinferno_b200.cache.manager import (REC_DRAWN, REC_LAST_TOKEN, REC_LENGTH, REC_SEED_HI, REC_SEED_LO,
                                                  REC_TEMPERATURE, RECORD_WORDS)
    m = manager()
    slot = m.open("a", seed=(7 << 32) + 0xFFFFFFFE, temperature=0.75)
    index, value = m.drain_record_updates()
    assert sorted(index) == list(range(slot * RECORD_WORDS, (slot + 1) * RECORD_WORDS))
    words = dict(zip((i - slot * RECORD_WORDS for i in index), value))
    assert words[REC_LENGTH] == 0 and words[REC_LAST_TOKEN] == -1 and words[REC_DRAWN] == 0
    assert words[REC_SEED_LO] == -2 and words[REC_SEED_HI] == 7          # two signed halves
    assert struct.unpack("<f", struct.pack("<i", words[REC_TEMPERATURE]))[0] == 0.75
    assert m.drain_record_updates() == ([], [])
    m.set_record("a", REC_LENGTH, 5), m.set_record("a", REC_LENGTH, 9), m.set_record("a", REC_LAST_TOKEN, 3)
    assert m.drain_record_updates() == ([slot * RECORD_WORDS + REC_LENGTH, slot * RECORD_WORDS + REC_LAST_TOKEN], [9, 3])
    m.close("a")
    assert m.open("b", seed=1) == slot and len(m.drain_record_updates()[0]) == RECORD_WORDS
    with pytest.raises(CacheError):
        m.set_record("a", REC_LENGTH, 1)
    with pytest.raises(CacheError):
        m.set_record("b", RECORD_WORDS, 1)


def test_keys_and_values_of_different_widths_share_a_page():
    m = manager(specs=[CacheSpec(2, 16, value_dim=8), CacheSpec(2, 16), CacheSpec(1, 24, value_dim=0)], tensors=True)
    assert len(m.groups) == 3 and [g.pool.shape[-1] for g in m.groups] == [4 * 2 * 24, 4 * 2 * 32, 4 * 24]
    unequal, equal, keys_only = (m.kv_binding(i) for i in range(3))
    assert unequal.keys.shape == (8, 2, 4, 16) and unequal.values.shape == (8, 2, 4, 8) and unequal.pool.shape == (8, 4 * 2 * 24)
    assert equal.pool.shape == (8, 2, 2, 4, 16) and equal.keys.data_ptr() == equal.pool[:, 0].data_ptr()
    assert equal.values.data_ptr() == equal.pool[:, 1].data_ptr()
    assert keys_only.values is None and keys_only.keys.shape == (8, 1, 4, 24)
    unequal.keys.fill_(1.0), unequal.values.fill_(2.0)
    assert m.groups[0].pool[0].sum().item() == 8 * 4 * 2 * (16 * 1 + 8 * 2)     # the views cover the pages, once
    assert m.kv_bytes_per_token() == 4 * (2 * 24 + 2 * 32 + 24)
