"""Multi-process control plane: rank 0 owns the HTTP front and the authoritative scheduler decisions, the other ranks
follow it step by step.

Every rank holds a full :class:`~atlas_b200.engine.LLMEngine` (its shard of the weights, its own KV pool and a replica
of the scheduler).  The scheduler is deterministic given (a) the stream of request events, (b) the clock value used for
deadlines / the SLAI policy and (c) what was sampled, so only those three things travel, over a CPU (gloo) group that is
independent of the GPU collectives:

* ``begin_step``: the leader broadcasts ``StepPlan(events, now)`` — requests admitted / aborted / expired since the
  previous step and its monotonic clock; followers apply the events and schedule with the same ``now``.  All ranks now
  build the same batch and launch the same kernels and collectives.
* ``finish_step``: only the leader samples (grammar masks, logit processors, stop strings live there); it broadcasts
  ``StepOutcome(records, dt)`` — per scheduled item the rows kept, tokens appended and the finish reason — and the
  followers replay that onto their sequences.  ``dt`` feeds the speculative throughput gate identically everywhere.

While idle the leader sends a heartbeat plan every ``heartbeat_s`` so that a follower's bounded wait only expires when
the leader is really gone; a follower that times out, or a leader whose broadcast fails, poisons its communicator,
latches the process fault and stops (the API then answers 503).  Shutdown is an explicit plan.

Reference parity: the reference drives its workers with 32-bit command words broadcast over NCCL
(``crates/spark-model/src/model/impl_a2.rs:385-401``: decode / batched decode / prefill chunk / alloc slot / verify
K / MTP propose / checkpoint / shutdown) and polls for errors while idle (``crates/spark-comm/src/lib.rs:51-63``).
Here the plan is one pickled object per step on a CPU group, so GPU streams never carry control traffic and CUDA
graphs stay legal under TP/EP.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..sampling import SamplingParams
from ..sched.sequence import FinishReason
from ..utils import fault
from .comm import CommBackend, CommError


@dataclass
class StepPlan:
    events: List[tuple] = field(default_factory=list)     # ("add", rid, prompt, sampling_dict, extras) | ("abort", rid, reason)
    now: float = 0.0
    shutdown: bool = False
    heartbeat: bool = False


@dataclass
class StepOutcome:
    records: Dict[int, Tuple[int, List[int], Optional[str]]] = field(default_factory=dict)   # item -> (rows kept, tokens, finish)
    dt: float = 0.0


class Shutdown(Exception):
    """Raised on a follower when the leader announced the end of service."""


class StepControl:
    """Glue between one engine and the control group.  ``comm`` only needs ``broadcast_object`` (a gloo
    ``TorchDistBackend`` in production, ``FakeComm`` in tests)."""

    def __init__(self, comm: CommBackend, heartbeat_s: float = 1.0):
        self.comm = comm
        self.is_leader = comm.rank == 0
        self.heartbeat_s = heartbeat_s
        self._pending: List[tuple] = []
        self._lock = threading.Lock()
        self._last_send = time.monotonic()
        self.plans_sent = 0

    # ------------------------------------------------------------------ leader side: event capture
    def note_add(self, rid: str, prompt: List[int], sampling: SamplingParams, extras: Dict[str, Any]) -> None:
        with self._lock:
            self._pending.append(("add", rid, list(prompt), sampling.to_dict(), dict(extras)))

    def note_abort(self, rid: str, reason: str = "abort") -> None:
        with self._lock:
            self._pending.append(("abort", rid, reason))

    def note_adapter(self, op: str, name: str, path: str = "") -> None:
        with self._lock:
            self._pending.append((op, name, path))

    def _bcast(self, obj):
        try:
            out = self.comm.broadcast_object(obj, src=0)
        except CommError as e:
            fault.latch(f"control plane: {e}")
            raise
        self._last_send = time.monotonic()
        return out

    # ------------------------------------------------------------------ per step
    def begin_step(self, engine) -> float:
        """Leader: expire deadlines, publish pending events.  Follower: receive and apply.  Returns the step clock."""
        if self.is_leader:
            now = time.monotonic()
            for s in engine.scheduler.expire(now):
                self.note_abort(s.request_id, "timeout")
            with self._lock:
                events, self._pending = self._pending, []
            # events that originate on the leader were already applied to its own engine when they were noted;
            # timeouts were applied by ``expire`` above
            self._bcast(StepPlan(events, now))
            self.plans_sent += 1
            return now
        while True:
            plan: StepPlan = self._bcast(None)
            if plan.shutdown:
                raise Shutdown()
            self.apply_events(engine, plan.events)
            if not plan.heartbeat:
                return plan.now

    def heartbeat(self) -> None:
        """Leader, while idle: keep followers' bounded waits alive."""
        if self.is_leader and time.monotonic() - self._last_send >= self.heartbeat_s:
            with self._lock:
                events, self._pending = self._pending, []
            self._bcast(StepPlan(events, time.monotonic(), heartbeat=True))

    def shutdown(self) -> None:
        if self.is_leader:
            self._bcast(StepPlan(shutdown=True))

    def finish_step(self, outcome: Optional[StepOutcome]) -> StepOutcome:
        return self._bcast(outcome if self.is_leader else None)

    # ------------------------------------------------------------------ follower side
    @staticmethod
    def apply_events(engine, events: List[tuple]) -> None:
        for ev in events:
            if ev[0] == "add":
                _, rid, prompt, sp, extras = ev
                engine.add_request(prompt, SamplingParams.from_dict(sp), request_id=rid, timeout_s=0, **extras)
            elif ev[0] == "abort":
                reason = FinishReason.TIMEOUT if ev[2] == "timeout" else FinishReason.ABORT
                engine.scheduler.abort(ev[1], reason)
                engine._seqs.pop(ev[1], None)
            elif ev[0] == "lora_load":          # every rank reads the adapter itself and keeps its own slices
                engine.load_adapter(ev[1], ev[2])
            elif ev[0] == "lora_unload":
                engine.unload_adapter(ev[1])


class DistributedEngine:
    """What the server talks to on rank 0 and what :func:`worker_loop` drives elsewhere."""

    def __init__(self, engine, control: StepControl):
        self.engine, self.control = engine, control
        engine.control = control

    def __getattr__(self, name):
        return getattr(self.engine, name)

    def add_request(self, prompt_tokens, sampling: Optional[SamplingParams] = None, request_id: Optional[str] = None,
                    namespace=0, priority: int = 0, timeout_s: Optional[float] = None, grammar: Any = None,
                    logits_processors=None, disable_spec: bool = False, stop_checker=None, adapter_slot: int = 0,
                    needs_full_logits: bool = False) -> str:
        assert self.control.is_leader, "requests enter on rank 0"
        sampling = sampling or SamplingParams()
        rid = self.engine.add_request(prompt_tokens, sampling, request_id, namespace, priority, timeout_s, grammar,
                                      logits_processors, disable_spec, stop_checker, adapter_slot)
        self.control.note_add(rid, [int(t) for t in prompt_tokens], sampling,
                              {"namespace": namespace, "priority": priority, "disable_spec": disable_spec,
                               "adapter_slot": adapter_slot,
                               "needs_full_logits": bool(needs_full_logits or grammar is not None or logits_processors)})
        return rid

    def abort(self, request_id: str) -> bool:
        ok = self.engine.abort(request_id)
        if ok:
            self.control.note_abort(request_id)
        return ok

    def load_adapter(self, name: str, path: str) -> int:
        """Adapter events travel in order with the request events, so a request that names the slot returned here
        reaches every follower after the adapter did."""
        slot = self.engine.load_adapter(name, path)
        self.control.note_adapter("lora_load", name, path)
        return slot

    def unload_adapter(self, name: str) -> None:
        self.engine.unload_adapter(name)
        self.control.note_adapter("lora_unload", name)

    def step(self):
        return self.engine.step()

    def idle(self) -> None:
        self.control.heartbeat()

    def shutdown(self) -> None:
        self.control.shutdown()


def worker_loop(engine, control: StepControl, max_steps: Optional[int] = None) -> int:
    """Follower main loop: block (bounded by the group timeout) for the next plan, run the step, repeat."""
    engine.control = control
    n = 0
    try:
        while max_steps is None or n < max_steps:
            engine.step()
            n += 1
    except Shutdown:
        pass
    return n


def make_control(timeout_s: float = 30.0, heartbeat_s: float = 1.0) -> StepControl:
    """A gloo group over the already-initialised default process group (any backend)."""
    import datetime

    import torch.distributed as dist

    from .comm import TorchDistBackend
    group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    return StepControl(TorchDistBackend(group, timeout_s), heartbeat_s)
