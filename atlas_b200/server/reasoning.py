"""Reasoning ("thinking") handling: splitting ``<think>...</think>`` from visible content while streaming, and a
logits processor that closes the think block once its token budget is spent.

Reference parity: ``crates/spark-server/src/reasoning_parser/*``, ``api/chat/thinking.rs``,
``scheduler/logit_processors/forced_think_end.rs``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple


class ReasoningSplitter:
    """Incremental splitter.  ``push(delta)`` returns ``(reasoning_delta, content_delta)``."""

    def __init__(self, open_tag: str = "<think>", close_tag: str = "</think>", starts_in_reasoning: bool = False):
        self.open, self.close = open_tag, close_tag
        self.in_reasoning = starts_in_reasoning
        self.seen_any = starts_in_reasoning
        self.done = False
        self._eat_newlines = False
        self.buf = ""

    def _hold(self, tag: str) -> int:
        for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
            if self.buf.endswith(tag[:k]):
                return k
        return 0

    def push(self, delta: str) -> Tuple[str, str]:
        self.buf += delta
        r_out, c_out = "", ""
        while True:
            if self.done:
                if self._eat_newlines:          # newlines right after the close tag belong to neither part
                    self.buf = self.buf.lstrip("\n")
                    if self.buf:
                        self._eat_newlines = False
                c_out += self.buf
                self.buf = ""
                return r_out, c_out
            if self.in_reasoning:
                i = self.buf.find(self.close)
                if i >= 0:
                    r_out += self.buf[:i]
                    self.buf = self.buf[i + len(self.close):]
                    self.in_reasoning, self.done, self._eat_newlines = False, True, True
                    continue
                h = self._hold(self.close)
                r_out += self.buf[:len(self.buf) - h]
                self.buf = self.buf[len(self.buf) - h:]
                return r_out, c_out
            # not yet in reasoning: the block may only open at the very start of the message
            stripped = self.buf.lstrip()
            if not self.seen_any and stripped.startswith(self.open):
                self.buf = stripped[len(self.open):]
                self.in_reasoning = self.seen_any = True
                continue
            if not self.seen_any and self.open.startswith(stripped) and stripped != self.open:
                return r_out, c_out         # could still become the open tag
            self.done = True

    def finish(self) -> Tuple[str, str]:
        out = self.buf
        self.buf = ""
        return (out, "") if self.in_reasoning else ("", out)


def split_reasoning(text: str, starts_in_reasoning: bool = False) -> Tuple[Optional[str], str]:
    sp = ReasoningSplitter(starts_in_reasoning=starts_in_reasoning)
    r, c = sp.push(text)
    r2, c2 = sp.finish()
    r, c = r + r2, c + c2
    return (r.strip() or None), c


class ThinkingBudget:
    """Logits processor: once ``budget`` tokens were generated inside the think block, force the close tag."""

    def __init__(self, close_ids: List[int], budget: int, open_ids: Optional[List[int]] = None,
                 starts_in_reasoning: bool = True):
        self.close_ids, self.budget = list(close_ids), budget
        self.starts = starts_in_reasoning
        self.forcing_at: Optional[int] = None

    def __call__(self, row, seq):
        out = seq.output_tokens
        n = len(out)
        k = len(self.close_ids)
        closed = any(out[i:i + k] == self.close_ids for i in range(0, max(0, n - k + 1)))
        if closed or not self.starts:
            return row
        if self.forcing_at is None and n >= self.budget:
            self.forcing_at = n
        if self.forcing_at is not None:
            j = n - self.forcing_at
            if 0 <= j < k:
                forced = self.close_ids[j]
                keep = row[forced].clone()
                row.fill_(float("-inf"))
                row[forced] = keep if keep > float("-inf") else 0.0
        return row
