"""Host-memory tier for the KV cache: a preempted decode keeps its computed KV blocks (and, for hybrid models, its
recurrent state) in pinned host memory instead of recomputing its whole context on resume.

The scheduler owns the bookkeeping (which sequence holds which host blocks) through the small allocator interface of
:class:`HostKVTier` (``num_free`` / ``alloc`` / ``free``); the engine performs the copies it lists in
``SchedulerOutput.swap_out`` / ``swap_in`` on the compute stream before the step's forward pass, swap-outs first, so a
device block that changes hands inside one step is saved before its new owner writes it, and host blocks are only
returned to the free list after the copy that reads them has been issued.

Sized by ``--swap-space-gb``.  Reference behaviour replaced: ``crates/spark-runtime/src/kv_host_tier/`` (arena + restore),
``crates/spark-server/src/scheduler/preempt.rs`` and ``restore_queue.rs`` (swap instead of recompute, parked restores).
"""
from __future__ import annotations

import os
import tempfile
from typing import Dict, List, Optional

import torch


def _raw(t: torch.Tensor) -> torch.Tensor:
    """8-bit float tensors are moved as bytes (indexing kernels do not exist for every float8 type)."""
    return t.view(torch.uint8) if t.element_size() == 1 else t


class DiskKVTier:
    """File-backed block store below the host tier: one fixed-size record per KV block (all layers' K and V slices of
    that block back to back), written and read with positional I/O on one preallocated file.  Parked sequences whose
    turn to resume is furthest away are spilled here when the host tier is full and come back through host blocks.
    Reference behaviour replaced: ``crates/avarok-tier/src/direct_swap`` (swap file) and the NVMe tier of
    ``crates/spark-storage/src/high_speed_swap.rs``."""

    def __init__(self, record_bytes: int, num_records: int, directory: str = ""):
        self.record_bytes, self.num_records = int(record_bytes), int(num_records)
        fd, self.path = tempfile.mkstemp(prefix="atlas_kv_swap_", suffix=".bin", dir=directory or None)
        self.fd = fd
        os.ftruncate(fd, self.record_bytes * self.num_records)
        self._free: List[int] = list(range(self.num_records - 1, -1, -1))
        self.records_out = 0
        self.records_in = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        assert n <= len(self._free), "disk tier exhausted"
        return [self._free.pop() for _ in range(n)]

    def free(self, ids: List[int]) -> None:
        self._free.extend(ids)

    def write(self, rec: int, data: bytes) -> None:
        assert len(data) == self.record_bytes
        os.pwrite(self.fd, data, rec * self.record_bytes)
        self.records_out += 1

    def read(self, rec: int) -> bytes:
        self.records_in += 1
        return os.pread(self.fd, self.record_bytes, rec * self.record_bytes)

    def close(self) -> None:
        if self.fd is not None:
            os.close(self.fd)
            self.fd = None
            try:
                os.unlink(self.path)
            except OSError:
                pass

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HostKVTier:
    def __init__(self, cache, num_host_blocks: int, num_state_slots: int = 0, disk_gb: float = 0.0, disk_dir: str = ""):
        self.cache = cache
        self.num_blocks = int(num_host_blocks)
        self._free: List[int] = list(range(self.num_blocks - 1, -1, -1))
        pin = any(k.is_cuda for k, _ in cache.kv.values())
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        for l, (k, v) in cache.kv.items():
            self.k[l] = torch.empty((self.num_blocks,) + tuple(k.shape[1:]), dtype=k.dtype, pin_memory=pin)
            self.v[l] = torch.empty((self.num_blocks,) + tuple(v.shape[1:]), dtype=v.dtype, pin_memory=pin)
        self.num_state_slots = int(num_state_slots) if cache.states else 0
        self._free_states: List[int] = list(range(self.num_state_slots - 1, -1, -1))
        self.states: Dict[int, Dict[str, torch.Tensor]] = {}
        for l, st in cache.states.items():
            self.states[l] = {name: torch.empty((self.num_state_slots,) + tuple(t.shape[1:]), dtype=t.dtype, pin_memory=pin)
                              for name, t in st.items() if name in ("conv", "h")}
        self.blocks_out = 0
        self.blocks_in = 0
        self.record_bytes = sum(k[0].numel() * k.element_size() + v[0].numel() * v.element_size() for k, v in cache.kv.values())
        self.disk: Optional[DiskKVTier] = None
        if disk_gb > 0 and self.record_bytes > 0:
            n_rec = int(disk_gb * (1 << 30)) // self.record_bytes
            if n_rec > 0:
                self.disk = DiskKVTier(self.record_bytes, n_rec, disk_dir)

    # ------------------------------------------------------------------ allocator (scheduler side)
    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_free_states(self) -> int:
        return len(self._free_states)

    def alloc(self, n: int) -> List[int]:
        assert n <= len(self._free), "host tier exhausted"
        return [self._free.pop() for _ in range(n)]

    def free(self, ids: List[int]) -> None:
        self._free.extend(ids)
        assert len(self._free) <= self.num_blocks, "host block freed twice"

    def alloc_state(self) -> int:
        return self._free_states.pop()

    def free_state(self, slot: Optional[int]) -> None:
        if slot is not None:
            self._free_states.append(slot)

    # ------------------------------------------------------------------ host <-> disk (engine side)
    def spill(self, host_blocks: List[int], disk_records: List[int]) -> None:
        """Host blocks -> disk records (the host blocks are free again afterwards; the scheduler accounts for that)."""
        for hb, rec in zip(host_blocks, disk_records):
            parts = []
            for l in self.k:
                parts.append(_raw(self.k[l][hb]).contiguous().view(torch.uint8).numpy().tobytes())
                parts.append(_raw(self.v[l][hb]).contiguous().view(torch.uint8).numpy().tobytes())
            self.disk.write(rec, b"".join(parts))

    def unspill(self, disk_records: List[int], host_blocks: List[int]) -> None:
        for rec, hb in zip(disk_records, host_blocks):
            data = memoryview(self.disk.read(rec))
            off = 0
            for l in self.k:
                for t in (self.k[l], self.v[l]):
                    n = t[hb].numel() * t.element_size()
                    flat = torch.frombuffer(bytearray(data[off:off + n]), dtype=torch.uint8)
                    t[hb].view(torch.uint8).reshape(-1).copy_(flat)
                    off += n

    # ------------------------------------------------------------------ copies (engine side)
    def copy_out(self, dev_blocks: List[int], host_blocks: List[int], state_slot: Optional[int] = None,
                 host_state: Optional[int] = None) -> None:
        assert len(dev_blocks) == len(host_blocks)
        if dev_blocks:
            hb = torch.tensor(host_blocks, dtype=torch.int64)
            for l, (k, v) in self.cache.kv.items():
                db = torch.tensor(dev_blocks, dtype=torch.int64, device=k.device)
                _raw(self.k[l])[hb] = _raw(k).index_select(0, db).to("cpu")
                _raw(self.v[l])[hb] = _raw(v).index_select(0, db).to("cpu")
            self.blocks_out += len(dev_blocks)
        if host_state is not None and state_slot is not None:
            for l, st in self.cache.states.items():
                for name, host in self.states[l].items():
                    host[host_state].copy_(st[name][state_slot])

    def copy_in(self, host_blocks: List[int], dev_blocks: List[int], host_state: Optional[int] = None,
                state_slot: Optional[int] = None) -> None:
        assert len(dev_blocks) == len(host_blocks)
        if dev_blocks:
            hb = torch.tensor(host_blocks, dtype=torch.int64)
            for l, (k, v) in self.cache.kv.items():
                db = torch.tensor(dev_blocks, dtype=torch.int64, device=k.device)
                _raw(k).index_copy_(0, db, _raw(self.k[l])[hb].to(k.device))
                _raw(v).index_copy_(0, db, _raw(self.v[l])[hb].to(v.device))
            self.blocks_in += len(dev_blocks)
        if host_state is not None and state_slot is not None:
            for l, st in self.cache.states.items():
                for name, host in self.states[l].items():
                    st[name][state_slot].copy_(host[host_state], non_blocking=True)
