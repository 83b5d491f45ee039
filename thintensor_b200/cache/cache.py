"""The cache of a model: a slot for each live sequence, keys and values for every run
of the schedule that keeps any, and per-sequence state of fixed size.

Runs with the same need (kv heads, head size, window) form a *group* with storage of
its own: one pool ``[runs, 2, blocks, kv_heads * block_tokens * head_dim]`` (keys at index
0 laid out ``[kv_heads, block_tokens, head_dim]`` inside a block, values at 1 laid out
transposed, ``[kv_heads, head_dim, block_tokens]``) and one block table, so that, say, windowed layers give blocks back
while full-attention layers keep theirs.  State needs are grouped the same way into
``[runs, slots, *shape]`` tensors, zeroed when a slot is handed out.

Freeing a slot returns its blocks to the pools; nothing is cleared, because attention
never reads beyond a sequence's length.  The reference's counterpart is PagedKVCache
(thinruntime/gpu_runtime.py:4132-4768) with per-layer windows at :4243-4253 and the
recurrent state tensors that live on its runtime object at :5466-5508.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import KVNeed, StateNeed
from .blocks import BlockPool, BlockTable, CacheError, SlotAllocator

BLOCK_TOKENS = 64


@dataclass
class KVGroup:
    need: KVNeed
    runs: list[int]                 # schedule entries that own a cache in this group
    table: BlockTable
    storage: torch.Tensor | None    # [runs, 2, blocks, kv_heads * BLOCK_TOKENS * head_dim]

    def bytes(self) -> int:
        return 0 if self.storage is None else self.storage.numel() * self.storage.element_size()


@dataclass
class StateGroup:
    need: StateNeed
    runs: list[int]
    storage: torch.Tensor | None    # [runs, slots, *shape]


@dataclass
class RunCache:
    """What one run of the schedule sees of the cache."""

    group: int | None               # index of its KV group, None if it keeps no keys
    k_pool: torch.Tensor | None     # [blocks, kv_heads, BLOCK_TOKENS, head_dim]
    v_pool: torch.Tensor | None     # [blocks, kv_heads, head_dim, BLOCK_TOKENS]
    writes: bool                    # False when the run reads another run's cache
    window: int | None


class SequenceCache:
    """Slots, block tables, pools and state for one model on one device.

    ``kv_needs[i]`` (None for nothing) and ``state_needs[i]`` (a list of StateNeed, or one, or
    None) are what run ``i`` of the schedule asks for (a run with several mixers has an entry
    for each of them); ``cache_from[i]`` names the entry whose keys entry ``i`` reads instead
    of keeping its own.  ``num_blocks`` blocks of 64 tokens are shared by all
    live sequences of a group; ``device=None`` keeps the bookkeeping only.
    """

    def __init__(self, kv_needs: list[KVNeed | None], state_needs: list, cache_from: list[int | None],
                 num_blocks: int, max_slots: int, dtype: torch.dtype, device: torch.device | str | None):
        self.block_tokens = BLOCK_TOKENS
        self.num_blocks = int(num_blocks)
        self.max_slots = int(max_slots)
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.slots = SlotAllocator(self.max_slots)
        self.lengths: dict[int, int] = {}           # live slot -> tokens cached
        self.kv_groups: list[KVGroup] = []
        self.state_groups: list[StateGroup] = []
        self._run_group: list[int | None] = [None] * len(kv_needs)
        self._run_index: list[int | None] = [None] * len(kv_needs)     # position in its group's storage
        self._run_state: list[list[tuple[int, int]]] = [[] for _ in kv_needs]
        self._cache_from = list(cache_from)

        by_need: dict[KVNeed, int] = {}
        for run, need in enumerate(kv_needs):
            if need is None or cache_from[run] is not None:
                continue
            if need not in by_need:
                by_need[need] = len(self.kv_groups)
                self.kv_groups.append(KVGroup(need, [], BlockTable(BlockPool(self.num_blocks), BLOCK_TOKENS, need.window), None))
            group = self.kv_groups[by_need[need]]
            self._run_group[run] = by_need[need]
            self._run_index[run] = len(group.runs)
            group.runs.append(run)
        for run, source in enumerate(cache_from):
            if source is None:
                continue
            if kv_needs[run] is None or kv_needs[source] is None:
                raise CacheError(f"run {run} reads the cache of run {source}, but one of them keeps no keys")
            a, b = kv_needs[run], kv_needs[source]
            if (a.kv_heads, a.head_dim) != (b.kv_heads, b.head_dim):
                raise CacheError(f"run {run} reads the cache of run {source}, whose key/value shape differs")
            if b.window is not None and (a.window is None or a.window > b.window):
                # the source's group gives blocks back by the source's window; a reader that looks
                # further back would meet blocks that are gone
                raise CacheError(f"run {run} reads the cache of run {source}, which keeps only the last {b.window} tokens, "
                                 f"but wants {'all of them' if a.window is None else 'the last ' + str(a.window)}")
            self._run_group[run] = self._run_group[source]
            self._run_index[run] = self._run_index[source]

        by_state: dict[StateNeed, int] = {}
        for run, needs in enumerate(state_needs):
            needs = [] if needs is None else ([needs] if isinstance(needs, StateNeed) else list(needs))
            for need in needs:
                if need not in by_state:
                    by_state[need] = len(self.state_groups)
                    self.state_groups.append(StateGroup(need, [], None))
                group = self.state_groups[by_state[need]]
                self._run_state[run].append((by_state[need], len(group.runs)))     # a run may hold several states of one shape
                group.runs.append(run)

        if self.device is not None:
            for group in self.kv_groups:
                shape = (len(group.runs), 2, self.num_blocks, group.need.kv_heads * BLOCK_TOKENS * group.need.head_dim)
                # zeros, not empty: a tensor-core product multiplies the unused tail of a block by a
                # probability of exactly zero, which must not meet a NaN left in fresh memory
                group.storage = torch.zeros(shape, dtype=dtype, device=self.device)
            for sgroup in self.state_groups:
                shape = (len(sgroup.runs), self.max_slots, *sgroup.need.shape)
                sgroup.storage = torch.zeros(shape, dtype=sgroup.need.dtype, device=self.device)

    # ---------------------------------------------------------------- slots
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        for group in self.kv_groups:
            group.table.open(slot)
        for sgroup in self.state_groups:
            if sgroup.storage is not None:
                sgroup.storage[:, slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)  # raises if it is not live
        del self.lengths[slot]
        for group in self.kv_groups:
            group.table.close(slot)

    def length(self, slot: int) -> int:
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is not live")
        return self.lengths[slot]

    # --------------------------------------------------------------- blocks
    def blocks_needed(self, slot: int, total_tokens: int) -> int:
        """Blocks (summed over groups, the worst group counted) that ``reserve`` would take."""
        return max((g.table.blocks_needed(slot, total_tokens) for g in self.kv_groups), default=0)

    def reserve(self, slot: int, total_tokens: int) -> None:
        """Make room for the sequence to grow to ``total_tokens`` tokens."""
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is not live")
        for group in self.kv_groups:
            group.table.reserve(slot, total_tokens)

    def advance(self, slot: int, new_tokens: int) -> None:
        """Record that ``new_tokens`` were appended; windowed groups give back blocks
        that no later token will read."""
        self.lengths[slot] += new_tokens
        for group in self.kv_groups:
            group.table.trim(slot, self.lengths[slot])

    def table_rows(self, group: int, slots: list[int], width: int) -> list[list[int]]:
        """The block-table rows of ``slots`` padded with -1 to ``width`` entries."""
        table = self.kv_groups[group].table
        rows = []
        for slot in slots:
            row = table.row(slot)
            if len(row) > width:
                raise CacheError(f"slot {slot} holds {len(row)} blocks, more than the table width {width}")
            rows.append(row + [-1] * (width - len(row)))
        return rows

    def max_blocks(self, slots: list[int]) -> int:
        return max((len(g.table.row(s)) for g in self.kv_groups for s in slots), default=0)

    # ---------------------------------------------------------------- views
    def run_cache(self, run: int) -> RunCache:
        group = self._run_group[run]
        if group is None:
            return RunCache(None, None, None, False, None)
        g = self.kv_groups[group]
        index = self._run_index[run]
        k = v = None
        if g.storage is not None:
            need = g.need
            k = g.storage[index, 0].view(self.num_blocks, need.kv_heads, BLOCK_TOKENS, need.head_dim)
            v = g.storage[index, 1].view(self.num_blocks, need.kv_heads, need.head_dim, BLOCK_TOKENS)
        return RunCache(group, k, v, self._cache_from[run] is None, g.need.window)

    def run_state(self, run: int) -> list[torch.Tensor]:
        """The state tensors of entry ``run``, each ``[slots, *shape]``, in the order it declared
        them (empty without a device or without states)."""
        out = []
        for group, index in self._run_state[run]:
            storage = self.state_groups[group].storage
            if storage is not None:
                out.append(storage[index])
        return out

    def bytes(self) -> int:
        total = sum(g.bytes() for g in self.kv_groups)
        for sgroup in self.state_groups:
            if sgroup.storage is not None:
                total += sgroup.storage.numel() * sgroup.storage.element_size()
        return total

    @property
    def free_blocks(self) -> int:
        return min((g.table.pool.free_count for g in self.kv_groups), default=self.num_blocks)
