"""Memory watchdog and preflight reserve check.

A daemon thread samples free device memory (``torch.cuda.mem_get_info``), available host memory and the KV pool's free
blocks.  Crossing the SOFT floor asks the engine to stop admitting new prefills until memory recovers (decodes keep
running so blocks drain); crossing the HARD floor trips the process-wide fault latch with an out-of-memory reason, so
the HTTP layer answers 503 and a supervisor restarts the process before the allocator fails inside a kernel launch
sequence.  ``preflight`` is the load-time form: refuse to start when weights + KV pool + a reserve cannot fit.

Decisions are a pure function of a sample (``decide``), so tests drive them with fake samples; nothing here allocates
or frees device memory.

Reference parity: ``crates/spark-runtime/src/cuda_backend.rs:613-625`` (watchdog thread polling free device memory),
``crates/spark-server/src/serve_phases/preflight.rs`` (memory reserve), ``serve_load.rs:493-510``.
"""
from __future__ import annotations

import enum
import threading
import time
from dataclasses import dataclass
from typing import Callable, Optional


class Level(enum.Enum):
    OK = "ok"
    SOFT = "soft"          # pause admission
    HARD = "hard"          # trip the fault latch


@dataclass
class MemorySample:
    device_free: int            # bytes
    device_total: int
    host_available: int         # bytes (0 = unknown)
    kv_free_blocks: int = 0
    kv_total_blocks: int = 0


@dataclass
class WatchdogConfig:
    soft_device_free: int = 2 << 30          # below this: no new prefills
    hard_device_free: int = 256 << 20        # below this: fault
    soft_host_available: int = 4 << 30
    hard_host_available: int = 512 << 20
    recover_factor: float = 1.5              # leave SOFT only once free memory exceeds soft * factor (hysteresis)
    interval_s: float = 0.5


def decide(s: MemorySample, cfg: WatchdogConfig, current: Level = Level.OK) -> Level:
    if s.device_total and s.device_free < cfg.hard_device_free:
        return Level.HARD
    if s.host_available and s.host_available < cfg.hard_host_available:
        return Level.HARD
    soft_dev = cfg.soft_device_free * (cfg.recover_factor if current == Level.SOFT else 1.0)
    soft_host = cfg.soft_host_available * (cfg.recover_factor if current == Level.SOFT else 1.0)
    if s.device_total and s.device_free < soft_dev:
        return Level.SOFT
    if s.host_available and s.host_available < soft_host:
        return Level.SOFT
    return Level.OK


def default_sampler(engine=None) -> MemorySample:
    import torch
    free = total = 0
    if torch.cuda.is_available():
        free, total = torch.cuda.mem_get_info()
    host = 0
    try:
        import psutil
        host = int(psutil.virtual_memory().available)
    except Exception:
        pass
    kv_free = kv_total = 0
    if engine is not None:
        kv_free, kv_total = engine.pool.num_free, engine.pool.num_blocks
    return MemorySample(int(free), int(total), host, kv_free, kv_total)


class MemoryWatchdog:
    def __init__(self, cfg: Optional[WatchdogConfig] = None, sampler: Callable[[], MemorySample] = default_sampler,
                 on_soft: Optional[Callable[[bool], None]] = None, on_hard: Optional[Callable[[str], None]] = None):
        self.cfg = cfg or WatchdogConfig()
        self.sampler, self.on_soft, self.on_hard = sampler, on_soft, on_hard
        self.level = Level.OK
        self.samples = 0
        self.last: Optional[MemorySample] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def poll(self) -> Level:
        """One sample + the callbacks its level change calls for (also what the thread runs)."""
        s = self.sampler()
        self.last = s
        self.samples += 1
        new = decide(s, self.cfg, self.level)
        if new != self.level:
            old, self.level = self.level, new
            if new == Level.HARD:
                if self.on_hard is not None:
                    self.on_hard(f"out of memory: device free {s.device_free >> 20} MiB of {s.device_total >> 20} MiB, "
                                 f"host available {s.host_available >> 20} MiB")
            elif self.on_soft is not None and (new == Level.SOFT) != (old == Level.SOFT):
                self.on_soft(new == Level.SOFT)
        return self.level

    def start(self) -> "MemoryWatchdog":
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="atlas-memory-watchdog", daemon=True)
            self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.cfg.interval_s):
            try:
                if self.poll() == Level.HARD:
                    return                      # the latch is one shot; nothing left to watch
            except Exception:
                pass

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None


def attach(engine, cfg: Optional[WatchdogConfig] = None) -> MemoryWatchdog:
    """Watchdog wired to an engine: SOFT pauses prefill admission in its scheduler, HARD trips the fault latch."""
    from .fault import FAULT_LATCH as LATCH

    def soft(on: bool) -> None:
        engine.scheduler.admission_paused = on

    return MemoryWatchdog(cfg, lambda: default_sampler(engine), soft, lambda why: LATCH.trip(why))


def preflight(weight_bytes: int, kv_bytes: int, device_free: int, reserve_bytes: int = 2 << 30) -> Optional[str]:
    """None when the plan fits, else a one-line reason (load-time check before any large allocation)."""
    need = weight_bytes + kv_bytes + reserve_bytes
    if need > device_free:
        return (f"needs {need >> 20} MiB (weights {weight_bytes >> 20} + KV {kv_bytes >> 20} + reserve {reserve_bytes >> 20}) "
                f"but only {device_free >> 20} MiB of device memory is free")
    return None
