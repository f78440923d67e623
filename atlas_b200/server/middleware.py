"""Auth (bearer tokens) and per-identity token-bucket rate limiting.

Reference parity: ``crates/spark-server/src/auth.rs``, ``rate_limiter.rs``, ``main_modules/middleware.rs``.
"""
from __future__ import annotations

import hmac
import threading
import time
from typing import Dict, Iterable, Optional


class BearerAuth:
    def __init__(self, tokens: Optional[Iterable[str]] = None):
        self.tokens = [t for t in (tokens or []) if t]

    @property
    def enabled(self) -> bool:
        return bool(self.tokens)

    def identity(self, authorization: Optional[str], x_api_key: Optional[str] = None) -> Optional[str]:
        """The matched token (the caller's identity) or None."""
        cand = None
        if authorization and authorization.lower().startswith("bearer "):
            cand = authorization[7:].strip()
        elif x_api_key:
            cand = x_api_key.strip()
        if cand is None:
            return None
        for t in self.tokens:
            if hmac.compare_digest(t, cand):
                return t
        return None


class TokenBucket:
    def __init__(self, rate_per_s: float, burst: float):
        self.rate, self.burst = rate_per_s, burst
        self.level, self.t = burst, time.monotonic()

    def take(self, n: float = 1.0, now: Optional[float] = None) -> bool:
        now = time.monotonic() if now is None else now
        self.level = min(self.burst, self.level + (now - self.t) * self.rate)
        self.t = now
        if self.level >= n:
            self.level -= n
            return True
        return False


class RateLimiter:
    def __init__(self, requests_per_minute: float = 0.0, burst: Optional[float] = None):
        self.rpm = requests_per_minute
        self.burst = burst if burst is not None else max(1.0, requests_per_minute / 6.0)
        self._b: Dict[str, TokenBucket] = {}
        self._lock = threading.Lock()

    @property
    def enabled(self) -> bool:
        return self.rpm > 0

    def allow(self, identity: str, now: Optional[float] = None) -> bool:
        if not self.enabled:
            return True
        with self._lock:
            b = self._b.get(identity)
            if b is None:
                b = self._b[identity] = TokenBucket(self.rpm / 60.0, self.burst)
            return b.take(1.0, now)
