"""Lightweight tracing: per-phase wall timers for the step loop, an optional launch trace of this engine's kernel
entry points, and a Chrome-trace (``chrome://tracing`` / Perfetto) export.  Everything is off unless enabled
(``serve --profile`` or ``ATLAS_TRACE=1``); when off, ``phase()`` is a shared no-op context manager.

Reference parity: ``crates/spark-runtime/src/launch_trace.rs`` (per-launch records), ``run_metrics.rs``,
``crates/spark-server/src/scheduler/mtp_timing.rs`` (phase timers), ``--profile``.
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from collections import defaultdict, deque
from typing import Any, Deque, Dict, List, Optional


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NULL = _Null()


class Tracer:
    def __init__(self, capacity: int = 65536):
        self.enabled = os.environ.get("ATLAS_TRACE", "0") not in ("0", "", "false")
        self.events: Deque[tuple] = deque(maxlen=capacity)           # (name, category, t_start_us, dur_us, tid, args)
        self.totals: Dict[str, List[float]] = defaultdict(lambda: [0.0, 0])   # name -> [seconds, count]
        self.launches: Dict[str, int] = defaultdict(int)
        self._lock = threading.Lock()
        self._t0 = time.perf_counter()

    # ------------------------------------------------------------------ control
    def enable(self, on: bool = True) -> None:
        self.enabled = on

    def reset(self) -> None:
        with self._lock:
            self.events.clear()
            self.totals.clear()
            self.launches.clear()
            self._t0 = time.perf_counter()

    # ------------------------------------------------------------------ recording
    def phase(self, name: str, category: str = "step", **args):
        """``with tracer.phase("schedule"): ...``"""
        if not self.enabled:
            return _NULL
        return self._span(name, category, args)

    @contextlib.contextmanager
    def _span(self, name: str, category: str, args: Dict[str, Any]):
        t = time.perf_counter()
        try:
            yield self
        finally:
            d = time.perf_counter() - t
            with self._lock:
                self.events.append((name, category, (t - self._t0) * 1e6, d * 1e6, threading.get_ident() & 0xFFFF, args))
                tot = self.totals[name]
                tot[0] += d
                tot[1] += 1

    def launch(self, entry: str) -> None:
        """Called by the kernel binding for every launching call when tracing is on."""
        if self.enabled:
            self.launches[entry] += 1
            self.events.append((entry, "launch", (time.perf_counter() - self._t0) * 1e6, 0.0, 0, {}))

    # ------------------------------------------------------------------ reporting
    def summary(self) -> Dict[str, Any]:
        with self._lock:
            phases = {k: {"seconds": round(v[0], 6), "count": v[1], "mean_ms": round(1e3 * v[0] / max(1, v[1]), 4)}
                      for k, v in sorted(self.totals.items(), key=lambda kv: -kv[1][0])}
            return {"enabled": self.enabled, "phases": phases, "launches": dict(self.launches)}

    def chrome_trace(self) -> Dict[str, Any]:
        with self._lock:
            evs = [{"name": n, "cat": c, "ph": "X" if d > 0 else "i", "ts": ts, "dur": d, "pid": os.getpid(), "tid": tid,
                    "args": a, **({"s": "t"} if d == 0 else {})} for n, c, ts, d, tid, a in self.events]
        return {"traceEvents": evs, "displayTimeUnit": "ms"}

    def dump(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.chrome_trace(), f)


TRACER = Tracer()


def phase(name: str, category: str = "step", **args):
    return TRACER.phase(name, category, **args)
