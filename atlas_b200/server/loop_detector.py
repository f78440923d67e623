"""Degenerate-loop guard: ends a generation whose output has fallen into a short cycle.

A greedy (or low-temperature) decode that starts repeating a phrase will keep doing so until ``max_tokens``; every such
token costs a full decode step and is worthless to the client.  The detector is a per-request stop checker (the engine
calls it after every appended token): the tail of the output is tested for exact periodicity, i.e. the last ``span``
tokens (at least ``min_repeats`` periods) repeat with some period ``p <= max_period``.  Checks run every ``stride``
tokens and cost ``O(max_period * span)`` comparisons in the worst case, with an early exit on the first mismatch of each
candidate period.

Reference behaviour replaced: ``crates/spark-server/src/loop_detector.rs`` (n-gram cycle detection on the decode stream;
the SimHash variant for near-duplicate paragraphs in ``loop_simhash.rs`` is not reproduced).
"""
from __future__ import annotations

from typing import Optional, Sequence


class LoopDetector:
    def __init__(self, span: int = 128, max_period: int = 64, min_repeats: int = 4, stride: int = 8):
        assert span >= 8 and max_period >= 1 and min_repeats >= 2 and stride >= 1
        self.span, self.max_period, self.min_repeats, self.stride = span, max_period, min_repeats, stride
        self.period: Optional[int] = None        # set when a loop was found

    @staticmethod
    def periodic_tail(toks: Sequence[int], period: int, length: int) -> bool:
        """True when the last ``length`` tokens satisfy ``t[i] == t[i - period]``."""
        n = len(toks)
        if length > n or period >= length:
            return False
        for i in range(1, length - period + 1):
            if toks[n - i] != toks[n - i - period]:
                return False
        return True

    def check(self, toks: Sequence[int]) -> Optional[int]:
        n = len(toks)
        if n < self.span:
            return None
        for p in range(1, self.max_period + 1):
            need = max(self.span, p * self.min_repeats)
            if n >= need and toks[-1] == toks[-1 - p] and self.periodic_tail(toks, p, need):
                return p
        return None

    def __call__(self, seq) -> bool:
        toks = seq.output_tokens
        if len(toks) % self.stride:
            return False
        p = self.check(toks)
        if p is not None:
            self.period = p
            return True
        return False
