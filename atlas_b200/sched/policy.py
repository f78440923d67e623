"""Admission-order policies.

* ``fifo``  – arrival order, head-of-line blocking (a request that does not fit stops admission).
* ``slai``  – shortest-prompt-first among waiting requests, no head-of-line blocking, and the prefill
  token budget shrinks when running decodes are close to their time-between-tokens deadline.

Reference parity: ``crates/spark-server/src/scheduling_policy.rs:31`` (``trait SchedulingPolicy``: FIFO / SLAI).
"""
from __future__ import annotations

from typing import List


class SchedulingPolicy:
    name = "base"
    head_of_line_blocking = True

    def order(self, waiting: List) -> List:
        return waiting

    def prefill_budget(self, max_prefill_tokens: int, num_decodes: int, since_last_decode_s: float) -> int:
        return max_prefill_tokens


class FifoPolicy(SchedulingPolicy):
    name = "fifo"

    def order(self, waiting: List) -> List:
        # preempted sequences sit at the front of the deque already; keep arrival order otherwise
        return waiting


class SlaiPolicy(SchedulingPolicy):
    name = "slai"
    head_of_line_blocking = False

    def __init__(self, tbt_deadline_ms: float = 100.0):
        self.tbt_deadline_s = tbt_deadline_ms / 1e3

    def order(self, waiting: List) -> List:
        return sorted(waiting, key=lambda s: (-s.priority, s.num_uncomputed, s.arrival))

    def prefill_budget(self, max_prefill_tokens: int, num_decodes: int, since_last_decode_s: float) -> int:
        if num_decodes == 0:
            return max_prefill_tokens
        slack = max(0.0, 1.0 - since_last_decode_s / self.tbt_deadline_s)
        # keep at least one block-sized chunk flowing so prefills cannot starve
        return max(256, int(max_prefill_tokens * slack))


def make_policy(name: str, tbt_deadline_ms: float = 100.0) -> SchedulingPolicy:
    name = (name or "fifo").lower()
    if name == "fifo":
        return FifoPolicy()
    if name == "slai":
        return SlaiPolicy(tbt_deadline_ms)
    raise ValueError(f"unknown scheduling policy '{name}' (fifo | slai)")
