"""Host-memory tier for the KV cache: a preempted decode keeps its computed KV blocks (and, for hybrid models, its
recurrent state) in pinned host memory instead of recomputing its whole context on resume.

The scheduler owns the bookkeeping (which sequence holds which host blocks) through the small allocator interface of
:class:`HostKVTier` (``num_free`` / ``alloc`` / ``free``); the engine performs the copies it lists in
``SchedulerOutput.swap_out`` / ``swap_in`` before the step's forward pass, swap-outs first, so a device block that
changes hands inside one step is saved before its new owner writes it, and host blocks are only returned to the free
list after the copy that reads them has been issued.  The copies themselves run on the tier's own stream (see
:class:`HostKVTier`); the step only waits for the on-device gather / scatter, not for the PCIe transfers.

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
    that block back to back), written and read on one preallocated file: batches of records through one io_uring
    submission straight from / into the pinned host rows (``csrc/runtime/uring_io.cpp``), plain positional I/O where
    io_uring is not available (or ``ATLAS_DISK_TIER_URING=0``).  Parked sequences whose
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

    def _uring(self):
        """The batched native path (``csrc/runtime/uring_io.cpp``) when the runtime library and io_uring are there."""
        if getattr(self, "_uring_ok", None) is None:
            try:
                from .. import runtime_native
                self._uring_ok = runtime_native.uring_available() and os.environ.get("ATLAS_DISK_TIER_URING", "1") != "0"
                self._rt = runtime_native
            except Exception:
                self._uring_ok = False
        return self._uring_ok

    def write_many(self, recs: List[int], rows: List[torch.Tensor]) -> None:
        """Host rows (one contiguous uint8 tensor of ``record_bytes`` each) -> records, all requests queued at once."""
        if recs and self._uring():
            try:
                self._rt.uring_rw(self.fd, True, [r * self.record_bytes for r in recs], [t.data_ptr() for t in rows], self.record_bytes)
                self.records_out += len(recs)
                return
            except OSError:
                self._uring_ok = False            # e.g. a filesystem that refuses the request type: plain I/O from now on
        for rec, t in zip(recs, rows):
            self.write(rec, t.numpy().tobytes())

    def read_many(self, recs: List[int], rows: List[torch.Tensor]) -> None:
        """Records -> host rows, read in place (no intermediate bytes objects on the batched path)."""
        if recs and self._uring():
            try:
                self._rt.uring_rw(self.fd, False, [r * self.record_bytes for r in recs], [t.data_ptr() for t in rows], self.record_bytes)
                self.records_in += len(recs)
                return
            except OSError:
                self._uring_ok = False
        for rec, t in zip(recs, rows):
            t.copy_(torch.frombuffer(bytearray(self.read(rec)), dtype=torch.uint8))

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
    """Pinned host pool of fixed-size records: record ``hb`` holds one KV block of every layer (K then V, layer after
    layer, the logical ``[block, head, dim]`` order of the pool views).

    Copies run on a dedicated CUDA stream and never block the host: a swap-out gathers the blocks of each layer into one
    device staging matrix (a handful of indexing kernels ordered after the compute stream by an event), then issues one
    device-to-host copy per record; the compute stream waits for the gather only, so the freed device blocks can be
    rewritten while the records are still travelling.  A swap-in is the mirror image (host-to-device copies into
    staging, scatter kernels, the compute stream waits for the scatter).  The single copy stream orders every use of a
    host record; the CPU only waits (``drain``) before it reads or writes records itself for the file tier."""

    def __init__(self, cache, num_host_blocks: int, num_state_slots: int = 0, disk_gb: float = 0.0, disk_dir: str = ""):
        self.cache = cache
        self.num_blocks = int(num_host_blocks)
        self._free: List[int] = list(range(self.num_blocks - 1, -1, -1))
        self.on_gpu = any(k.is_cuda for k, _ in cache.kv.values())
        self.device = next((k.device for k, _ in cache.kv.values()), torch.device("cpu"))
        # (layer, which, byte offset, bytes) of every slice of a record
        self.layout: List[tuple] = []
        off = 0
        for l, (k, v) in cache.kv.items():
            for which, t in (("k", k), ("v", v)):
                n = t[0].numel() * t.element_size()
                self.layout.append((l, which, off, n))
                off += n
        self.record_bytes = off
        self.pool = torch.empty(self.num_blocks, max(1, self.record_bytes), dtype=torch.uint8, pin_memory=self.on_gpu)
        self.num_state_slots = int(num_state_slots) if cache.states else 0
        self._free_states: List[int] = list(range(self.num_state_slots - 1, -1, -1))
        self.states: Dict[int, Dict[str, torch.Tensor]] = {}
        for l, st in cache.states.items():
            self.states[l] = {name: torch.empty((self.num_state_slots,) + tuple(t.shape[1:]), dtype=t.dtype, pin_memory=self.on_gpu)
                              for name, t in st.items() if name in ("conv", "h")}
        self.stream = torch.cuda.Stream(device=self.device) if self.on_gpu else None
        self._staging: Optional[torch.Tensor] = None
        self.blocks_out = 0
        self.blocks_in = 0
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

    def drain(self) -> None:
        """Wait until every issued copy has landed (before the CPU touches records)."""
        if self.stream is not None:
            self.stream.synchronize()

    # ------------------------------------------------------------------ host <-> disk (engine side)
    def spill(self, host_blocks: List[int], disk_records: List[int]) -> None:
        """Host records -> disk records (the host blocks are free again afterwards; the scheduler accounts for that)."""
        self.drain()
        self.disk.write_many(list(disk_records), [self.pool[hb] for hb in host_blocks])

    def unspill(self, disk_records: List[int], host_blocks: List[int]) -> None:
        self.drain()
        self.disk.read_many(list(disk_records), [self.pool[hb] for hb in host_blocks])

    # ------------------------------------------------------------------ copies (engine side)
    def _stage(self, n: int) -> torch.Tensor:
        if self._staging is None or self._staging.shape[0] < n:
            self._staging = torch.empty(max(n, 64), self.record_bytes, dtype=torch.uint8, device=self.device)
        return self._staging[:n]

    def _tensor(self, l: int, which: str) -> torch.Tensor:
        k, v = self.cache.kv[l]
        return k if which == "k" else v

    def copy_out(self, dev_blocks: List[int], host_blocks: List[int], state_slot: Optional[int] = None,
                 host_state: Optional[int] = None) -> None:
        assert len(dev_blocks) == len(host_blocks)
        n = len(dev_blocks)
        if self.on_gpu:
            cur = torch.cuda.current_stream(self.device)
            self.stream.wait_stream(cur)                      # the blocks' last writers have been issued on `cur`
            with torch.cuda.stream(self.stream):
                if n:
                    db = torch.tensor(dev_blocks, dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
                    st = self._stage(n)
                    for l, which, off, nbytes in self.layout:
                        t = self._tensor(l, which)
                        st[:, off:off + nbytes] = _raw(t).index_select(0, db).reshape(n, -1).view(torch.uint8)
                gathered = torch.cuda.Event()
                gathered.record(self.stream)
                for i, hb in enumerate(host_blocks):
                    self.pool[hb].copy_(st[i], non_blocking=True)
                if host_state is not None and state_slot is not None:
                    for l, stt in self.cache.states.items():
                        for name, host in self.states[l].items():
                            host[host_state].copy_(stt[name][state_slot], non_blocking=True)
                    gathered = torch.cuda.Event()
                    gathered.record(self.stream)
            cur.wait_event(gathered)                          # device blocks / state slot may be rewritten after this
        else:
            for i, (dbk, hb) in enumerate(zip(dev_blocks, host_blocks)):
                for l, which, off, nbytes in self.layout:
                    blk = self._tensor(l, which)[dbk].contiguous()
                    self.pool[hb, off:off + nbytes] = _raw(blk).reshape(-1).view(torch.uint8)
            if host_state is not None and state_slot is not None:
                for l, stt in self.cache.states.items():
                    for name, host in self.states[l].items():
                        host[host_state].copy_(stt[name][state_slot])
        self.blocks_out += n

    def copy_in(self, host_blocks: List[int], dev_blocks: List[int], host_state: Optional[int] = None,
                state_slot: Optional[int] = None) -> None:
        assert len(dev_blocks) == len(host_blocks)
        n = len(dev_blocks)
        if self.on_gpu:
            cur = torch.cuda.current_stream(self.device)
            self.stream.wait_stream(cur)                      # earlier readers of the destination blocks are on `cur`
            with torch.cuda.stream(self.stream):
                if n:
                    db = torch.tensor(dev_blocks, dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
                    st = self._stage(n)
                    for i, hb in enumerate(host_blocks):
                        st[i].copy_(self.pool[hb], non_blocking=True)
                    for l, which, off, nbytes in self.layout:
                        t = self._tensor(l, which)
                        src = st[:, off:off + nbytes].contiguous().view(_raw(t).dtype).view((n,) + tuple(t.shape[1:]))
                        _raw(t).index_copy_(0, db, src)
                if host_state is not None and state_slot is not None:
                    for l, stt in self.cache.states.items():
                        for name, host in self.states[l].items():
                            stt[name][state_slot].copy_(host[host_state], non_blocking=True)
                done = torch.cuda.Event()
                done.record(self.stream)
            cur.wait_event(done)
        else:
            for hb, dbk in zip(host_blocks, dev_blocks):
                for l, which, off, nbytes in self.layout:
                    t = self._tensor(l, which)
                    src = self.pool[hb, off:off + nbytes].clone().view(_raw(t).dtype).view(tuple(t.shape[1:]))
                    _raw(t)[dbk] = src
            if host_state is not None and state_slot is not None:
                for l, stt in self.cache.states.items():
                    for name, host in self.states[l].items():
                        stt[name][state_slot].copy_(host[host_state])
        self.blocks_in += n
