"""Engine counters and latency summaries (exported through ``/metrics`` and the scheduler snapshot).

Reference parity: ``crates/spark-server/src/metrics.rs`` (``atlas_requests_total``,
``atlas_time_to_first_token_seconds``, ``atlas_generation_tokens_total`` ...) and
``scheduler/snapshot.rs``.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, field
from typing import Dict, List


class Reservoir:
    """Bounded sample store with exact percentiles over what it holds."""

    def __init__(self, cap: int = 4096):
        self.cap, self._v, self.count, self.total = cap, [], 0, 0.0

    def add(self, x: float) -> None:
        self.count += 1
        self.total += x
        if len(self._v) >= self.cap:
            self._v.pop(0)
        self._v.append(x)

    def percentile(self, p: float) -> float:
        if not self._v:
            return 0.0
        s = sorted(self._v)
        i = min(len(s) - 1, max(0, int(round(p / 100.0 * (len(s) - 1)))))
        return s[i]

    @property
    def mean(self) -> float:
        return self.total / self.count if self.count else 0.0


@dataclass
class EngineStats:
    requests_total: int = 0
    requests_finished: int = 0
    generation_tokens: int = 0
    prompt_tokens: int = 0
    steps: int = 0
    decode_steps: int = 0
    prefill_tokens: int = 0
    spec_proposed: int = 0
    spec_accepted: int = 0
    busy_time_s: float = 0.0
    ttft: Reservoir = field(default_factory=Reservoir)
    step_time: Reservoir = field(default_factory=Reservoir)
    tokens_per_s_ema: float = 0.0

    def on_first_token(self, ttft_s: float) -> None:
        self.ttft.add(ttft_s)

    def on_step(self, dt: float, out, emitted: int) -> None:
        self.steps += 1
        self.busy_time_s += dt
        self.step_time.add(dt)
        n_dec = sum(1 for i in out.items if i.is_decode)
        if n_dec:
            self.decode_steps += 1
        self.prefill_tokens += sum(i.num_tokens for i in out.items if not i.is_decode and not i.verify_drafts)
        if dt > 0:
            inst = emitted / dt
            self.tokens_per_s_ema = inst if self.tokens_per_s_ema == 0 else 0.9 * self.tokens_per_s_ema + 0.1 * inst

    def as_dict(self) -> Dict[str, float]:
        return {"requests_total": self.requests_total, "requests_finished": self.requests_finished,
                "generation_tokens": self.generation_tokens, "steps": self.steps, "decode_steps": self.decode_steps,
                "prefill_tokens": self.prefill_tokens, "spec_proposed": self.spec_proposed,
                "spec_accepted": self.spec_accepted, "busy_time_s": self.busy_time_s,
                "ttft_p50_s": self.ttft.percentile(50), "ttft_p90_s": self.ttft.percentile(90),
                "step_p50_s": self.step_time.percentile(50), "tokens_per_s": self.tokens_per_s_ema}
