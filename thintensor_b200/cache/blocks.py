"""Host-side bookkeeping of the cache: which sequence slots are live and which blocks
of the pool each of them holds.  Pure Python, no device: every decision the cache makes
can be tested without a GPU.

The reference has one sequence per cache object, keeps its pages in per-layer Python
lists and returns them to a free list on ``reset(reuse_pages=True)``
(thinruntime/gpu_runtime.py:4255-4273, 4520-4528).  Here many sequences share one pool
of fixed-size blocks; a sequence's blocks are named by its row of a block table.
"""
from __future__ import annotations


class CacheError(RuntimeError):
    """The cache was asked for something it cannot give (no free slot, no free block,
    a slot that is not live)."""


class SlotAllocator:
    """Slots 0..n-1; a slot is live between ``alloc`` and ``free``."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise CacheError(f"a cache needs at least one slot, got {num_slots}")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))  # pop() hands out the lowest first
        self._live: set[int] = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"all {self.num_slots} sequence slots are in use")
        slot = self._free.pop()
        self._live.add(slot)
        return slot

    def free(self, slot: int) -> None:
        if slot not in self._live:
            raise CacheError(f"slot {slot} is not live (freed twice, or never allocated)")
        self._live.remove(slot)
        self._free.append(slot)

    def is_live(self, slot: int) -> bool:
        return slot in self._live

    @property
    def live(self) -> frozenset[int]:
        return frozenset(self._live)

    @property
    def free_count(self) -> int:
        return len(self._free)


class BlockPool:
    """Block ids 0..n-1 of one storage pool."""

    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise CacheError(f"a block pool needs at least one block, got {num_blocks}")
        self.num_blocks = num_blocks
        self._free = list(range(num_blocks - 1, -1, -1))
        self._held = [False] * num_blocks

    def alloc(self, count: int) -> list[int]:
        if count > len(self._free):
            raise CacheError(
                f"the cache is full: {count} more blocks are needed and {len(self._free)} of {self.num_blocks} are free"
            )
        out = [self._free.pop() for _ in range(count)]
        for block in out:
            self._held[block] = True
        return out

    def free(self, blocks: list[int]) -> None:
        for block in blocks:
            if not 0 <= block < self.num_blocks or not self._held[block]:
                raise CacheError(f"block {block} is not held (freed twice, or never allocated)")
            self._held[block] = False
            self._free.append(block)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.num_blocks - len(self._free)


class BlockTable:
    """The blocks of every live slot in one storage group, in logical order.  Entry
    ``i`` of a slot's row holds tokens ``i * block_tokens .. (i + 1) * block_tokens - 1``;
    ``-1`` marks a block that a windowed group has already given back."""

    def __init__(self, pool: BlockPool, block_tokens: int, window: int | None = None):
        self.pool = pool
        self.block_tokens = block_tokens
        self.window = window
        self.rows: dict[int, list[int]] = {}

    def open(self, slot: int) -> None:
        if slot in self.rows:
            raise CacheError(f"slot {slot} already has a block table row")
        self.rows[slot] = []

    def reserve(self, slot: int, tokens: int) -> bool:
        """Make room for positions 0..tokens-1; returns whether the row changed."""
        row = self.rows[slot]
        need = -(-tokens // self.block_tokens)
        if need <= len(row):
            return False
        row.extend(self.pool.alloc(need - len(row)))
        return True

    def blocks_needed(self, slot: int, tokens: int) -> int:
        return max(0, -(-tokens // self.block_tokens) - len(self.rows[slot]))

    def trim(self, slot: int, length: int) -> bool:
        """For a windowed group: give back the blocks whose every token is older than
        the ``window`` tokens that the next position will see."""
        if self.window is None:
            return False
        row = self.rows[slot]
        first_needed = max(0, length + 1 - self.window)  # oldest key the next token reads
        changed = False
        for i in range(min(first_needed // self.block_tokens, len(row))):
            if row[i] >= 0:
                self.pool.free([row[i]])
                row[i] = -1
                changed = True
        return changed

    def close(self, slot: int) -> None:
        row = self.rows.pop(slot)
        self.pool.free([b for b in row if b >= 0])

    def row(self, slot: int) -> list[int]:
        return self.rows[slot]
