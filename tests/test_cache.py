"""The cache's bookkeeping without a device: no slot or block lost, held twice or freed
twice; groups with storage of their own; windows give blocks back; state is declared."""
from __future__ import annotations

import random

import pytest
import torch

from thintensor_b200.cache import BlockPool, BlockTable, CacheError, SequenceCache, SlotAllocator
from thintensor_b200.parts.base import KVNeed, StateNeed


def test_slots_are_never_held_twice_or_freed_twice():
    slots = SlotAllocator(3)
    a, b, c = slots.alloc(), slots.alloc(), slots.alloc()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheError, match="in use"):
        slots.alloc()
    slots.free(b)
    with pytest.raises(CacheError, match="not live"):
        slots.free(b)
    with pytest.raises(CacheError, match="not live"):
        slots.free(17)
    assert slots.alloc() == b and slots.free_count == 0 and slots.live == frozenset({0, 1, 2})


def test_block_pool_accounting_under_random_use():
    pool = BlockPool(50)
    rng = random.Random(0)
    held: list[list[int]] = []
    for _ in range(2000):
        if held and (rng.random() < 0.5 or pool.free_count == 0):
            pool.free(held.pop(rng.randrange(len(held))))
        else:
            held.append(pool.alloc(rng.randint(1, min(5, pool.free_count))))
        flat = [b for group in held for b in group]
        assert len(flat) == len(set(flat)) == pool.held_count            # nothing held twice
        assert pool.held_count + pool.free_count == 50                   # nothing lost
    with pytest.raises(CacheError, match="cache is full"):
        pool.alloc(pool.free_count + 1)
    block = pool.alloc(1)
    pool.free(block)
    with pytest.raises(CacheError, match="not held"):
        pool.free(block)


def test_block_table_reserve_and_close():
    pool = BlockPool(10)
    table = BlockTable(pool, 64)
    table.open(0)
    assert table.reserve(0, 1) and len(table.row(0)) == 1
    assert not table.reserve(0, 64) and table.reserve(0, 65) and len(table.row(0)) == 2
    assert table.blocks_needed(0, 64 * 5) == 3
    table.open(1)
    table.reserve(1, 64 * 8)
    with pytest.raises(CacheError, match="cache is full"):
        table.reserve(0, 64 * 3)
    table.close(1)
    assert pool.free_count == 8
    with pytest.raises(CacheError):
        table.open(0)


def test_window_gives_blocks_back():
    pool = BlockPool(10)
    table = BlockTable(pool, 64, window=100)
    table.open(0)
    table.reserve(0, 400)
    assert pool.held_count == 7
    assert table.trim(0, 400)             # the next token (position 400) reads keys 301..400: blocks 0..3 go
    assert table.row(0)[:4] == [-1] * 4 and all(b >= 0 for b in table.row(0)[4:])
    assert pool.held_count == 3 and not table.trim(0, 400)
    table.close(0)
    assert pool.free_count == 10


def make_cache(num_blocks=8, max_slots=3):
    full, windowed = KVNeed(2, 16), KVNeed(2, 16, window=64)
    kv = [full, windowed, full, None, full]
    state = [None, None, None, StateNeed((4, 2)), None]
    source = [None, None, None, None, 0]       # the last run reads the first run's keys
    return SequenceCache(kv, state, source, num_blocks, max_slots, torch.float32, None)


def test_groups_have_storage_of_their_own():
    cache = make_cache()
    assert [g.runs for g in cache.kv_groups] == [[0, 2], [1]]
    assert [g.runs for g in cache.state_groups] == [[3]]
    first, shared, none = cache.run_cache(0), cache.run_cache(4), cache.run_cache(3)
    assert first.group == shared.group == 0 and first.writes and not shared.writes
    assert none.group is None and cache.run_cache(1).window == 64
    with pytest.raises(CacheError, match="keeps no keys"):
        SequenceCache([None, KVNeed(1, 16)], [None, None], [None, 0], 4, 2, torch.float32, None)


def test_a_reader_may_not_look_further_back_than_its_source_keeps():
    """A run that reads another run's cache sees what that run's group keeps: blocks that have slid out
    of the source's window are given back, so a reader without a window, or with a wider one, is refused;
    a narrower window (or the same) is fine."""
    windowed, full = KVNeed(2, 16, window=128), KVNeed(2, 16)
    for reader in (full, KVNeed(2, 16, window=256)):
        with pytest.raises(CacheError, match="keeps only the last 128 tokens"):
            SequenceCache([windowed, reader], [None, None], [None, 0], 8, 2, torch.float32, None)
    for reader in (windowed, KVNeed(2, 16, window=64)):
        cache = SequenceCache([windowed, reader], [None, None], [None, 0], 8, 2, torch.float32, None)
        assert cache.run_cache(1).group == cache.run_cache(0).group and not cache.run_cache(1).writes
    cache = SequenceCache([full, windowed], [None, None], [None, 0], 8, 2, torch.float32, None)     # a window onto a full cache
    slot = cache.alloc_slot()
    cache.reserve(slot, 400)
    cache.advance(slot, 400)
    assert all(b >= 0 for b in cache.table_rows(0, [slot], 7)[0]), "the full source keeps every block"


def test_sequences_come_and_go():
    cache = make_cache(num_blocks=8, max_slots=3)
    a, b = cache.alloc_slot(), cache.alloc_slot()
    cache.reserve(a, 130)
    cache.advance(a, 130)
    cache.reserve(b, 64)
    cache.advance(b, 64)
    assert cache.length(a) == 130 and cache.max_blocks([a, b]) == 3
    assert cache.kv_groups[0].table.pool.held_count == 4
    assert cache.kv_groups[1].table.pool.held_count == 3      # the windowed group gave back the block that slid out
    rows = cache.table_rows(0, [b, a], 4)
    assert rows[0][1:] == [-1, -1, -1] and all(x >= 0 for x in rows[1][:3]) and rows[1][3] == -1
    with pytest.raises(CacheError, match="more than the table width"):
        cache.table_rows(0, [a], 2)
    cache.free_slot(a)
    with pytest.raises(CacheError, match="not live"):
        cache.free_slot(a)
    with pytest.raises(CacheError, match="not live"):
        cache.length(a)
    c = cache.alloc_slot()
    assert c == a and cache.length(c) == 0                    # the slot is used again, empty
    cache.free_slot(b)
    cache.free_slot(c)
    assert cache.free_blocks == 8 and cache.slots.free_count == 3
    with pytest.raises(CacheError, match="cache is full"):
        d = cache.alloc_slot()
        cache.reserve(d, 64 * 9)


def test_workspace_zeroes_its_zeroed_buffers_again():
    """Buffers handed out zeroed (tickets, flags) are left zero by their users; after a kernel that gave up they are
    zeroed again, and only they."""
    import torch

    from thintensor_b200.engine.context import Workspace

    workspace = Workspace(torch.device("cpu"))
    flags = workspace.get_zeroed("flags", (16,), torch.int32)
    plain = workspace.get("scratch", (16,), torch.int32)
    assert int(flags.abs().sum()) == 0
    flags[3] = 1
    plain.fill_(7)
    workspace.zero_again()
    assert int(flags.abs().sum()) == 0 and int(plain.sum()) == 7 * 16
    assert workspace.get_zeroed("flags", (16,), torch.int32).data_ptr() == flags.data_ptr()       # still the same memory
