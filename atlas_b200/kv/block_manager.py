"""Paged-KV block bookkeeping (host side).

A pool of fixed-size blocks with reference counts: a block allocated to a sequence starts at 1,
sharing it through the prefix cache increments it, and it returns to the free list at 0.  When the
native runtime library is built the same interface is served by the C++ ``BlockPool``
(``csrc/runtime/block_pool.cpp``); this Python class is the portable implementation and the oracle
for it.

Reference parity: ``crates/spark-runtime/src/kv_cache.rs:417`` (``PagedKvCache``),
``kv_cache/paged_impl.rs`` (``free_blocks`` + ``block_ref_counts``).
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Iterable, List, Optional


class OutOfBlocks(RuntimeError):
    pass


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int):
        self.num_blocks, self.block_size = int(num_blocks), int(block_size)
        self._free: Deque[int] = deque(range(self.num_blocks))
        self._ref = [0] * self.num_blocks
        self.high_water = 0

    # -------------------------------------------------------------- queries
    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_blocks - len(self._free)

    def ref_count(self, block: int) -> int:
        return self._ref[block]

    def blocks_for_tokens(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size

    # -------------------------------------------------------------- mutation
    def alloc(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise OutOfBlocks(f"need {n} blocks, {len(self._free)} free")
        out = [self._free.popleft() for _ in range(n)]
        for b in out:
            self._ref[b] = 1
        self.high_water = max(self.high_water, self.num_used)
        return out

    def inc_ref(self, blocks: Iterable[int]) -> None:
        for b in blocks:
            if self._ref[b] <= 0:
                raise ValueError(f"inc_ref on free block {b}")
            self._ref[b] += 1

    def free(self, blocks: Iterable[int]) -> int:
        """Drop one reference from each block; returns how many actually returned to the free list."""
        released = 0
        for b in blocks:
            r = self._ref[b]
            if r <= 0:
                raise ValueError(f"double free of block {b}")
            self._ref[b] = r - 1
            if r == 1:
                self._free.append(b)
                released += 1
        return released

    def check_invariants(self) -> None:
        free = set(self._free)
        assert len(free) == len(self._free), "duplicate block in free list"
        for b in range(self.num_blocks):
            assert (self._ref[b] == 0) == (b in free), f"block {b}: ref {self._ref[b]} vs free {b in free}"


class SlotPool:
    """Fixed pool of recurrent-state slots (GDN ``h`` + conv window) with stable addresses so CUDA
    graphs can reference them (reference: ``crates/spark-model/src/model/ssm_pool.rs``)."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free: Deque[int] = deque(range(num_slots))

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> Optional[int]:
        return self._free.popleft() if self._free else None

    def free(self, slot: int) -> None:
        assert slot not in self._free
        self._free.append(slot)
