"""Process-wide GPU fault latch.

After any failed GPU operation the context is probed with a no-op synchronisation; a sticky error means
the CUDA context is lost for the rest of the process, which flips a one-shot latch.  The HTTP layer answers
503 while the latch is set and ``/health`` reports the fault (a supervisor restarts the process).

Reference parity: ``crates/avarok-core/src/fault.rs:1-60`` (``Fatality``, one-shot latch),
``crates/spark-runtime/src/cuda_backend/fault_probe.rs``, ``main_modules/middleware.rs:340-355``.
"""
from __future__ import annotations

import enum
import threading
import time
from typing import Callable, Optional

STICKY_MARKERS = ("illegal memory access", "illegal instruction", "unspecified launch failure", "device-side assert",
                  "misaligned address", "launch timed out", "context is destroyed", "an illegal", "uncorrectable",
                  "cuda error: ", "cudaerror")


class Fatality(enum.Enum):
    NONE = "none"
    REQUEST_SCOPED = "request_scoped"      # the op failed, the context still answers
    CONTEXT_LOST = "context_lost"


def classify_probe(op_failed: bool, probe_ok: bool) -> Fatality:
    """Pure classification of (the operation failed?, does a no-op sync still succeed?)."""
    if not op_failed:
        return Fatality.NONE
    return Fatality.REQUEST_SCOPED if probe_ok else Fatality.CONTEXT_LOST


def default_probe() -> bool:
    """True when the CUDA context still answers a synchronise."""
    try:
        import torch
        if not torch.cuda.is_available():
            return True
        torch.cuda.synchronize()
        return True
    except Exception:
        return False


class FaultLatch:
    def __init__(self, probe: Callable[[], bool] = default_probe):
        self._probe = probe
        self._lock = threading.Lock()
        self.tripped = False
        self.reason: Optional[str] = None
        self.when: Optional[float] = None
        self.request_scoped_failures = 0

    def observe_exception(self, exc: BaseException) -> Fatality:
        msg = str(exc).lower()
        looks_gpu = any(m in msg for m in STICKY_MARKERS) or exc.__class__.__name__ in ("AcceleratorError", "KernelError")
        if not looks_gpu:
            self.request_scoped_failures += 1
            return Fatality.REQUEST_SCOPED
        f = classify_probe(True, self._probe())
        if f is Fatality.CONTEXT_LOST:
            self.trip(f"{exc.__class__.__name__}: {exc}")
        else:
            self.request_scoped_failures += 1
        return f

    def observe_status_word(self, status: int) -> Fatality:
        """A kernel's bounded wait gave up (non-zero device status word): the context is fine, the step is not."""
        if status == 0:
            return Fatality.NONE
        self.request_scoped_failures += 1
        return Fatality.REQUEST_SCOPED

    def trip(self, reason: str) -> None:
        with self._lock:
            if not self.tripped:          # one-shot: the first reason sticks
                self.tripped, self.reason, self.when = True, reason, time.time()

    def reset_for_tests(self) -> None:
        with self._lock:
            self.tripped, self.reason, self.when, self.request_scoped_failures = False, None, None, 0


FAULT_LATCH = FaultLatch()


def latch(reason: str) -> None:
    """Trip the process-wide latch (non-GPU fatal conditions, e.g. a dead control plane, use this too)."""
    FAULT_LATCH.trip(reason)
