"""Collective backends behind one small interface.

* :class:`SingleGpuBackend` — world size 1, every call is a no-op (reference: ``SingleGpuBackend``,
  ``crates/spark-comm/src/lib.rs:177``).
* :class:`TorchDistBackend` — ``torch.distributed`` process group (NCCL on GPUs, gloo on CPU).  On GPUs this
  is the *baseline* path; the product path is :class:`atlas_b200.parallel.symm.SymmBackend`, whose
  all-reduce / reduce-scatter / all-to-all run inside this engine's own kernels over NVLink peer memory.
* :class:`FakeComm` — in-process simulated ranks for protocol tests: collectives rendezvous through a shared
  object, a rank can be told to fail or never join, waits are bounded.

Health: every backend carries an ``unhealthy`` flag set when a collective raises or times out; once poisoned,
further calls raise :class:`CommError` immediately (reference: ``poison_on_error``,
``crates/spark-comm/src/collective_wait.rs``; ``nccl_backend.rs:242-359``).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional, Sequence

import torch


class CommError(RuntimeError):
    pass


class CommBackend:
    rank: int = 0
    world_size: int = 1
    unhealthy: bool = False
    name = "base"

    def _guard(self) -> None:
        if self.unhealthy:
            raise CommError(f"{self.name}: communicator is poisoned by an earlier failure")

    def poison(self, why: str = "") -> None:
        self.unhealthy = True
        self.poison_reason = why

    # collectives (sum reductions)
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor: raise NotImplementedError
    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor: raise NotImplementedError
    def reduce_scatter(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor: raise NotImplementedError
    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor: raise NotImplementedError
    def all_to_all(self, parts: List[torch.Tensor]) -> List[torch.Tensor]: raise NotImplementedError
    def barrier(self) -> None: raise NotImplementedError
    def broadcast_object(self, obj, src: int = 0): raise NotImplementedError


class SingleGpuBackend(CommBackend):
    name = "single"

    def all_reduce(self, t): return t
    def all_gather(self, t, dim=0): return t
    def reduce_scatter(self, t, dim=0): return t
    def broadcast(self, t, src=0): return t
    def all_to_all(self, parts): return list(parts)
    def barrier(self): return None
    def broadcast_object(self, obj, src=0): return obj


class TorchDistBackend(CommBackend):
    """``torch.distributed`` group; also records per-collective call counts for diagnostics."""
    name = "torch.distributed"

    def __init__(self, group=None, timeout_s: float = 30.0):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.timeout_s = timeout_s
        self.calls: Dict[str, int] = {}

    def _run(self, what: str, fn: Callable):
        self._guard()
        self.calls[what] = self.calls.get(what, 0) + 1
        try:
            return fn()
        except Exception as e:  # a failed or timed-out collective poisons the communicator
            self.poison(f"{what}: {e}")
            raise CommError(f"{what} failed on rank {self.rank}: {e}") from e

    def all_reduce(self, t):
        self._run("all_reduce", lambda: self.dist.all_reduce(t, group=self.group))
        return t

    def all_reduce_async(self, t):
        """Starts the reduction and returns a handle whose ``wait()`` orders the current stream after it."""
        return self._run("all_reduce", lambda: self.dist.all_reduce(t, group=self.group, async_op=True))

    def all_gather(self, t, dim=0):
        def go():
            outs = [torch.empty_like(t) for _ in range(self.world_size)]
            self.dist.all_gather(outs, t.contiguous(), group=self.group)
            return torch.cat(outs, dim=dim)
        return self._run("all_gather", go)

    def reduce_scatter(self, t, dim=0):
        def go():
            chunks = [c.contiguous() for c in t.chunk(self.world_size, dim=dim)]
            out = torch.empty_like(chunks[0])
            self.dist.reduce_scatter(out, chunks, group=self.group)
            return out
        return self._run("reduce_scatter", go)

    def broadcast(self, t, src=0):
        self._run("broadcast", lambda: self.dist.broadcast(t, src=self.dist.get_global_rank(self.group, src) if self.group else src,
                                                           group=self.group))
        return t

    def all_to_all(self, parts):
        def go():
            # variable sizes: exchange row counts first
            dev = parts[0].device
            counts = torch.tensor([p.shape[0] for p in parts], dtype=torch.int64, device=dev)
            rc = torch.empty_like(counts)
            self.dist.all_to_all_single(rc, counts, group=self.group)
            tail, dt = tuple(parts[0].shape[1:]), parts[0].dtype
            outs = [torch.empty((int(n),) + tail, dtype=dt, device=dev) for n in rc.tolist()]
            self.dist.all_to_all(outs, [p.contiguous() for p in parts], group=self.group)
            return outs
        if self.dist.get_backend(self.group) == "gloo":
            return self._run("all_to_all", lambda: self._a2a_via_gather(parts))
        return self._run("all_to_all", go)

    def _a2a_via_gather(self, parts):
        gathered: List[Optional[list]] = [None] * self.world_size
        self.dist.all_gather_object(gathered, [p.cpu() for p in parts], group=self.group)
        return [gathered[r][self.rank].to(parts[0].device) for r in range(self.world_size)]

    def barrier(self):
        self._run("barrier", lambda: self.dist.barrier(group=self.group))

    def broadcast_object(self, obj, src=0):
        def go():
            box = [obj]
            self.dist.broadcast_object_list(box, src=src, group=self.group)
            return box[0]
        return self._run("broadcast_object", go)


# ----------------------------------------------------------------------------- in-process fake ranks
class FakeWorld:
    """Shared rendezvous for :class:`FakeComm` ranks running as threads of one process."""

    def __init__(self, world_size: int, timeout_s: float = 2.0):
        self.world_size, self.timeout_s = world_size, timeout_s
        self._cv = threading.Condition()
        self._slots: Dict[int, Dict[int, object]] = {}
        self._done: Dict[int, int] = {}
        self.dropped: set = set()          # (seq_no, rank) contributions to swallow, simulating a lost message
        self.dead: set = set()             # ranks that never join again

    def exchange(self, seq_no: int, rank: int, value):
        """All ranks deposit ``value`` under ``seq_no`` and get everyone's values; bounded wait."""
        with self._cv:
            if (seq_no, rank) not in self.dropped and rank not in self.dead:
                self._slots.setdefault(seq_no, {})[rank] = value
                self._cv.notify_all()
            deadline = time.monotonic() + self.timeout_s
            while len(self._slots.get(seq_no, {})) < self.world_size:
                left = deadline - time.monotonic()
                if left <= 0:
                    missing = sorted(set(range(self.world_size)) - set(self._slots.get(seq_no, {})))
                    raise CommError(f"collective #{seq_no} timed out on rank {rank}; missing ranks {missing}")
                self._cv.wait(left)
            vals = dict(self._slots[seq_no])
            self._done[seq_no] = self._done.get(seq_no, 0) + 1
            if self._done[seq_no] == self.world_size:
                del self._slots[seq_no], self._done[seq_no]
            return [vals[r] for r in range(self.world_size)]

    def comm(self, rank: int) -> "FakeComm":
        return FakeComm(self, rank)

    def run(self, fn, timeout_s: float = 120.0) -> list:
        """Run ``fn(rank)`` on one thread per rank; returns the results in rank order, re-raising the first error."""
        out, err = [None] * self.world_size, [None] * self.world_size

        def body(r):
            try:
                out[r] = fn(r)
            except BaseException as e:      # noqa: BLE001 - reported to the caller below
                err[r] = e

        ts = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(self.world_size)]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout_s)
        for e in err:
            if e is not None:
                raise e
        return out


class FakeComm(CommBackend):
    name = "fake"

    def __init__(self, world: FakeWorld, rank: int):
        self.world, self.rank, self.world_size = world, rank, world.world_size
        self._seq = 0
        self.log: List[str] = []

    def _x(self, what: str, value):
        self._guard()
        self._seq += 1
        self.log.append(what)
        try:
            return self.world.exchange(self._seq, self.rank, value)
        except CommError as e:
            self.poison(str(e))
            raise

    def all_reduce(self, t):
        vals = self._x("all_reduce", t.clone())
        out = vals[0].clone()
        for v in vals[1:]:
            out += v
        t.copy_(out)
        return t

    def all_gather(self, t, dim=0):
        return torch.cat(self._x("all_gather", t.clone()), dim=dim)

    def reduce_scatter(self, t, dim=0):
        vals = self._x("reduce_scatter", t.clone())
        tot = vals[0].clone()
        for v in vals[1:]:
            tot += v
        return tot.chunk(self.world_size, dim=dim)[self.rank].clone()

    def broadcast(self, t, src=0):
        vals = self._x("broadcast", t.clone())
        t.copy_(vals[src])
        return t

    def all_to_all(self, parts):
        vals = self._x("all_to_all", [p.clone() for p in parts])
        return [vals[r][self.rank] for r in range(self.world_size)]

    def barrier(self):
        self._x("barrier", None)

    def broadcast_object(self, obj, src=0):
        return self._x("broadcast_object", obj)[src]
