"""AsyncEngine: one OS thread owns the LLMEngine (and with it the CUDA context); HTTP handlers talk to it
through a thread-safe inbox and per-request asyncio queues.

Reference parity: the scheduler OS thread + ``tokio::mpsc<InferenceRequest>`` / per-request
``StreamEvent`` channels of ``crates/spark-server/src/scheduler/mod.rs:262-402``; drain-on-shutdown of
``scheduler/shutdown_drain.rs``; model hot-swap hand-over of ``main_modules/model_swap.rs``.
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Callable, Dict, List, Optional

from ..engine import LLMEngine, RequestOutput, RequestRejected
from ..sampling import SamplingParams
from ..utils.fault import FAULT_LATCH


@dataclass
class StreamEvent:
    """``kind``: token | done | error."""
    kind: str
    tokens: List[int] = field(default_factory=list)
    output: Optional[RequestOutput] = None
    error: str = ""
    logprobs: Optional[list] = None


class AsyncEngine:
    def __init__(self, engine: LLMEngine, idle_sleep_s: float = 0.002):
        self.engine = engine
        self._inbox: "queue.Queue[tuple]" = queue.Queue()
        self._streams: Dict[str, tuple] = {}          # request id -> (loop, asyncio.Queue)
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._draining = threading.Event()
        self._wake = threading.Event()
        self.idle_sleep_s = idle_sleep_s
        self.started_at = time.time()
        self.last_error: Optional[str] = None
        self.on_tick: Optional[Callable[[LLMEngine], None]] = None   # metrics / snapshot hook

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> None:
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="atlas-scheduler", daemon=True)
            self._thread.start()

    def shutdown(self, drain: bool = True, timeout_s: float = 30.0) -> None:
        if drain:
            self._draining.set()
            deadline = time.time() + timeout_s
            while self.engine.has_unfinished() and time.time() < deadline and self._thread and self._thread.is_alive():
                time.sleep(0.01)
        self._stop.set()
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None

    def swap_engine(self, new_engine: LLMEngine) -> None:
        """Model hot-swap: drain the scheduler, stop it, install the new engine, start again."""
        self.shutdown(drain=True)
        self.engine = new_engine
        self._stop.clear()
        self._draining.clear()
        self.start()

    @property
    def accepting(self) -> bool:
        return not self._draining.is_set() and not self._stop.is_set() and not FAULT_LATCH.tripped

    # ------------------------------------------------------------------ submission (called from asyncio handlers)
    async def generate(self, prompt_tokens: List[int], sampling: SamplingParams, request_id: Optional[str] = None,
                       **kw) -> AsyncIterator[StreamEvent]:
        if not self.accepting:
            raise RuntimeError("engine is not accepting requests")
        rid = request_id or "req-" + uuid.uuid4().hex[:16]
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        self._streams[rid] = (loop, q)
        self._inbox.put(("add", rid, prompt_tokens, sampling, kw))
        self._wake.set()
        try:
            while True:
                ev: StreamEvent = await q.get()
                yield ev
                if ev.kind in ("done", "error"):
                    return
        finally:
            if rid in self._streams:
                del self._streams[rid]
                self._inbox.put(("abort", rid))
                self._wake.set()

    def abort(self, request_id: str) -> None:
        self._inbox.put(("abort", request_id))
        self._wake.set()

    # ------------------------------------------------------------------ scheduler thread
    def _emit(self, rid: str, ev: StreamEvent) -> None:
        tgt = self._streams.get(rid)
        if tgt is None:
            return
        loop, q = tgt
        try:
            loop.call_soon_threadsafe(q.put_nowait, ev)
        except RuntimeError:
            pass        # the client's loop is gone

    def _drain_inbox(self) -> None:
        while True:
            try:
                msg = self._inbox.get_nowait()
            except queue.Empty:
                return
            if msg[0] == "add":
                _, rid, toks, sampling, kw = msg
                try:
                    self.engine.add_request(toks, sampling, request_id=rid, **kw)
                except (RequestRejected, ValueError) as e:
                    self._emit(rid, StreamEvent("error", error=str(e)))
            elif msg[0] == "abort":
                self.engine.abort(msg[1])

    def _run(self) -> None:
        eng = self.engine
        if eng.model.device.type == "cuda":
            import torch
            torch.cuda.set_device(eng.model.device)
        while not self._stop.is_set():
            self._drain_inbox()
            if not eng.has_unfinished():
                idle = getattr(eng, "idle", None)      # multi-process leader: heartbeat to the follower ranks
                if idle is not None:
                    idle()
                self._wake.wait(self.idle_sleep_s * 10)
                self._wake.clear()
                continue
            try:
                outs = eng.step()
            except Exception as e:     # classify: a sticky CUDA error trips the process-wide fault latch
                self.last_error = repr(e)
                FAULT_LATCH.observe_exception(e)
                for rid in list(self._streams):
                    self._emit(rid, StreamEvent("error", error=f"engine step failed: {e}"))
                if FAULT_LATCH.tripped:
                    return
                # request-scoped failure: drop everything that was in flight and keep serving
                for rid in list(eng._seqs):
                    eng.abort(rid)
                continue
            for o in outs:
                if o.new_tokens:
                    self._emit(o.request_id, StreamEvent("token", tokens=o.new_tokens,
                                                         logprobs=(o.logprobs[-len(o.new_tokens):] if o.logprobs else None)))
                if o.finished:
                    self._emit(o.request_id, StreamEvent("done", output=o))
            if self.on_tick is not None:
                self.on_tick(eng)
