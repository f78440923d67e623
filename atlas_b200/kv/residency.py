"""Generic two-level residency: an opaque key -> fixed-size blob page table over a bounded HOT tier (slots in RAM) and
an optionally capped COLD tier (fixed-stride records in a file or in memory).

* ``put`` never rejects: a full hot arena spills its coldest unpinned resident to the cold tier; a capped cold tier
  drops its coldest key (a later ``get`` of it is a clean miss).
* ``get`` of a cold key promotes it back to the hot tier (spilling another key if needed).
* Read pins: a slot that a reader holds is never chosen as a spill victim; ``unpin`` releases it.
* Replacement policy of the hot tier: ``lru`` or ``arc`` (adaptive replacement: two recency / frequency lists with
  ghost histories that tune the split, so a scan of one-time keys does not flush the frequently used ones).

The KV host tier, the prefix-snapshot store and the LoRA adapter pool all page through this one mechanism.

Reference parity: ``crates/avarok-tier/src/{residency,traits,mem,direct_swap}.rs`` (``SlotArena`` / ``SwapStore`` /
``Residency``: two-level LRU, read pins, never-reject puts).
"""
from __future__ import annotations

import os
from collections import OrderedDict
from typing import Dict, Hashable, List, Optional


class MemSwapStore:
    """Cold tier in RAM (tests, small deployments)."""

    def __init__(self, record_bytes: int, capacity: Optional[int] = None):
        self.record_bytes, self.capacity = record_bytes, capacity
        self._d: Dict[int, bytes] = {}
        self._free: List[int] = []
        self._next = 0

    def alloc(self) -> Optional[int]:
        if self._free:
            return self._free.pop()
        if self.capacity is not None and self._next >= self.capacity:
            return None
        self._next += 1
        return self._next - 1

    def free(self, rec: int) -> None:
        self._d.pop(rec, None)
        self._free.append(rec)

    def write(self, rec: int, blob: bytes) -> None:
        self._d[rec] = bytes(blob)

    def read(self, rec: int) -> bytes:
        return self._d[rec]


class FileSwapStore(MemSwapStore):
    """Cold tier as fixed-stride records of one file, positional I/O (no shared file offset between threads)."""

    def __init__(self, path: str, record_bytes: int, capacity: Optional[int] = None):
        super().__init__(record_bytes, capacity)
        self._fd = os.open(path, os.O_RDWR | os.O_CREAT, 0o600)

    def write(self, rec: int, blob: bytes) -> None:
        assert len(blob) <= self.record_bytes
        os.pwrite(self._fd, bytes(blob).ljust(self.record_bytes, b"\0"), rec * self.record_bytes)

    def read(self, rec: int) -> bytes:
        return os.pread(self._fd, self.record_bytes, rec * self.record_bytes)

    def close(self) -> None:
        os.close(self._fd)


class Residency:
    def __init__(self, num_slots: int, slot_bytes: int, cold=None, policy: str = "lru"):
        assert num_slots >= 1 and policy in ("lru", "arc")
        self.num_slots, self.slot_bytes, self.policy = num_slots, slot_bytes, policy
        self.cold = cold
        self._slots: List[Optional[bytes]] = [None] * num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._hot: Dict[Hashable, int] = {}                      # key -> slot
        self._pins: Dict[Hashable, int] = {}
        self._lru: "OrderedDict[Hashable, None]" = OrderedDict() # hot keys, coldest first (lru policy)
        self._cold: "OrderedDict[Hashable, int]" = OrderedDict() # key -> record, coldest first
        # ARC state: t1 recent-once, t2 frequent (both hot); b1 / b2 ghosts; p = target size of t1
        self._t1: "OrderedDict[Hashable, None]" = OrderedDict()
        self._t2: "OrderedDict[Hashable, None]" = OrderedDict()
        self._b1: "OrderedDict[Hashable, None]" = OrderedDict()
        self._b2: "OrderedDict[Hashable, None]" = OrderedDict()
        self._p = 0.0
        self.stats = {"hits": 0, "cold_hits": 0, "misses": 0, "spills": 0, "drops": 0}

    # ------------------------------------------------------------------ policy
    def _touch(self, key: Hashable, new: bool) -> None:
        if self.policy == "lru":
            self._lru.pop(key, None)
            self._lru[key] = None
            return
        if key in self._t1:
            del self._t1[key]
            self._t2[key] = None
        elif key in self._t2:
            self._t2.move_to_end(key)
        elif key in self._b1:                                    # a ghost hit in the recency history: grow t1's share
            self._p = min(float(self.num_slots), self._p + max(1.0, len(self._b2) / max(1, len(self._b1))))
            del self._b1[key]
            self._t2[key] = None
        elif key in self._b2:
            self._p = max(0.0, self._p - max(1.0, len(self._b1) / max(1, len(self._b2))))
            del self._b2[key]
            self._t2[key] = None
        else:
            self._t1[key] = None

    def _victim(self) -> Optional[Hashable]:
        if self.policy == "lru":
            return next((k for k in self._lru if not self._pins.get(k)), None)
        first, second = (self._t1, self._t2) if (len(self._t1) > self._p or not self._t2) else (self._t2, self._t1)
        for lst in (first, second):
            for k in lst:
                if not self._pins.get(k):
                    return k
        return None

    def _forget_hot(self, key: Hashable) -> None:
        self._lru.pop(key, None)
        if key in self._t1:
            del self._t1[key]
            self._b1[key] = None
        elif key in self._t2:
            del self._t2[key]
            self._b2[key] = None
        for g in (self._b1, self._b2):
            while len(g) > self.num_slots:
                g.popitem(last=False)

    # ------------------------------------------------------------------ tiers
    def _spill_one(self) -> bool:
        key = self._victim()
        if key is None:
            return False
        slot = self._hot.pop(key)
        blob = self._slots[slot]
        self._slots[slot] = None
        self._free.append(slot)
        self._forget_hot(key)
        if self.cold is not None:
            rec = self.cold.alloc()
            if rec is None and self._cold:                       # capped cold tier: its coldest key goes
                old, orec = self._cold.popitem(last=False)
                self.cold.free(orec)
                self.stats["drops"] += 1
                rec = self.cold.alloc()
            if rec is not None:
                self.cold.write(rec, blob)
                self._cold[key] = rec
                self.stats["spills"] += 1
                return True
        self.stats["drops"] += 1
        return True

    def _place(self, key: Hashable, blob: bytes) -> bool:
        if not self._free and not self._spill_one():
            return False                                         # every slot is pinned by a reader
        slot = self._free.pop()
        self._slots[slot] = bytes(blob)
        self._hot[key] = slot
        self._touch(key, True)
        return True

    # ------------------------------------------------------------------ API
    def put(self, key: Hashable, blob: bytes) -> None:
        assert len(blob) <= self.slot_bytes
        if key in self._hot:
            self._slots[self._hot[key]] = bytes(blob)
            self._touch(key, False)
            return
        if key in self._cold:
            self.cold.free(self._cold.pop(key))
        if not self._place(key, blob):
            # all slots pinned: the blob goes straight to the cold tier (or is dropped if there is none)
            if self.cold is not None:
                rec = self.cold.alloc()
                if rec is not None:
                    self.cold.write(rec, blob)
                    self._cold[key] = rec
                    return
            self.stats["drops"] += 1

    def get(self, key: Hashable, pin: bool = False) -> Optional[bytes]:
        slot = self._hot.get(key)
        if slot is not None:
            self.stats["hits"] += 1
            self._touch(key, False)
        elif key in self._cold:
            rec = self._cold.pop(key)
            blob = self.cold.read(rec)[:self.slot_bytes]
            self.cold.free(rec)
            self.stats["cold_hits"] += 1
            if not self._place(key, blob):
                rec2 = self.cold.alloc()
                self.cold.write(rec2, blob)
                self._cold[key] = rec2
                return blob
            slot = self._hot[key]
        else:
            self.stats["misses"] += 1
            return None
        if pin:
            self._pins[key] = self._pins.get(key, 0) + 1
        return self._slots[slot]

    def unpin(self, key: Hashable) -> None:
        n = self._pins.get(key, 0)
        if n <= 1:
            self._pins.pop(key, None)
        else:
            self._pins[key] = n - 1

    def remove(self, key: Hashable) -> None:
        slot = self._hot.pop(key, None)
        if slot is not None:
            self._slots[slot] = None
            self._free.append(slot)
            self._lru.pop(key, None)
            self._t1.pop(key, None)
            self._t2.pop(key, None)
        rec = self._cold.pop(key, None)
        if rec is not None:
            self.cold.free(rec)
        self._pins.pop(key, None)

    def __contains__(self, key: Hashable) -> bool:
        return key in self._hot or key in self._cold

    @property
    def hot_keys(self) -> List[Hashable]:
        return list(self._hot)

    @property
    def cold_keys(self) -> List[Hashable]:
        return list(self._cold)
