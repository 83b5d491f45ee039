"""The sequence cache: slots, block tables, key/value pools and per-sequence state."""
from .blocks import BlockPool, BlockTable, CacheError, SlotAllocator
from .cache import BLOCK_TOKENS, KVGroup, RunCache, SequenceCache, StateGroup

__all__ = ["BLOCK_TOKENS", "BlockPool", "BlockTable", "CacheError", "KVGroup", "RunCache", "SequenceCache", "SlotAllocator", "StateGroup"]
