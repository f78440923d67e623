"""Pre-sample logit stages around thinking and tool calls, as one per-request processor.

``ThinkToolPipeline`` is called by the sampler with ``(row, seq)`` like any other logits processor.  It follows the
sequence's output incrementally (inside / after the think block, tool call opened or not) and runs these stages in
order; each is a no-op when the token ids it needs are unknown (fail-open):

1. ``confidence``   inside thinking, after ``min_think_tokens``: a streak of ``streak`` tokens whose top-1 probability is
                    >= ``conf_p`` arms an early end of thinking (reads the logits, never changes them).
2. ``mid_word``     inside thinking: the close tag is not allowed right after a token that ends in a letter or digit
                    (closing there cuts a word in half); an armed early end waits for the same boundary.
3. ``forced_end``   an armed early end emits the close tag, token by token.
4. ``post_close``   after thinking ended: neither the close tag nor the open tag may appear again.
5. ``tool_in_think``inside thinking the tool-call opener is masked; outside, when the caller flagged a tool-call loop
                    (``suppress_tool_call``), it gets a strong negative bias instead of a mask so that overwhelming
                    evidence can still win.
6. ``pin_tool``     right after the close tag, when the request requires a tool call and none is open yet, the
                    tool-call opener is the only admissible continuation (token by token for multi-token openers).
7. ``margin``       (opt-in) observability only: counts positions whose top-1 / top-2 log-probability gap is below
                    ``low_margin`` (the regime where FP8 rounding can flip a greedy pick); never changes the logits.

Masks apply to single-token tags only (the special tokens of real tokenizers); a tag that takes several ordinary
tokens is never masked, because its first token is ordinary text.  Forced emissions work for any length.

Reference parity: ``crates/spark-server/src/scheduler/logit_processors/{mid_word,post_close,tool_during_think,
pin_tool_call,b1_margin,f2_confidence}.rs`` and the stage order of ``mod.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

NEG_INF = float("-inf")


@dataclass
class PipelineStats:
    positions: int = 0
    low_margin: int = 0
    mid_word_defers: int = 0
    post_close_masks: int = 0
    tool_masks: int = 0
    tool_biases: int = 0
    pinned_tool_calls: int = 0
    early_think_ends: int = 0
    min_gap: float = field(default=float("inf"))


def _ends_with(tokens: Sequence[int], tag: Sequence[int]) -> bool:
    k = len(tag)
    return k > 0 and len(tokens) >= k and list(tokens[-k:]) == list(tag)


class ThinkToolPipeline:
    def __init__(self, think_open: Sequence[int] = (), think_close: Sequence[int] = (), tool_open: Sequence[int] = (),
                 token_text: Optional[Callable[[int], str]] = None, starts_in_think: bool = False,
                 require_tool_call: bool = False, suppress_tool_call: bool = False, tool_loop_bias: float = -12.0,
                 min_think_tokens: int = 400, conf_p: float = 0.95, streak: int = 0, low_margin: float = 1.5,
                 margin: bool = False, guard_pinned: bool = False):
        self.open, self.close, self.tool = list(think_open), list(think_close), list(tool_open)
        self.token_text = token_text
        self.in_think = bool(starts_in_think)
        self.think_ended = False
        self.think_just_ended = False
        self.tool_opened = False
        self.require_tool_call = bool(require_tool_call)
        self.suppress_tool_call = bool(suppress_tool_call)
        self.tool_loop_bias = float(tool_loop_bias)
        self.min_think_tokens, self.conf_p, self.streak = int(min_think_tokens), float(conf_p), int(streak)
        self.low_margin = float(low_margin)
        # the two stages below read a value back from the row (a device synchronisation per token on a GPU), so they are
        # on only when asked for: the margin counter, and the check for a position another processor already pinned
        self.margin, self.guard_pinned = bool(margin), bool(guard_pinned)
        self.stats = PipelineStats()
        self._seen = 0                       # output tokens already folded into the state
        self._think_tokens = 0
        self._run = 0                        # current streak of confident tokens
        self.force_end_thinking = False
        self._forcing: Optional[List[int]] = None      # remaining ids of a forced tag
        self._pin_pending = False

    # ------------------------------------------------------------------ state
    def _advance(self, out: Sequence[int]) -> None:
        self.think_just_ended = False
        for i in range(self._seen, len(out)):
            upto = out[:i + 1]
            if self.in_think:
                self._think_tokens += 1
                if _ends_with(upto, self.close):
                    self.in_think, self.think_ended, self.think_just_ended = False, True, i == len(out) - 1
                    self._pin_pending = self.require_tool_call
            elif not self.think_ended and _ends_with(upto, self.open):
                self.in_think = True
            if not self.in_think and _ends_with(upto, self.tool):
                self.tool_opened = True
                self._pin_pending = False
        self._seen = len(out)

    def _mid_word(self, out: Sequence[int]) -> bool:
        if not out or self.token_text is None:
            return False
        text = self.token_text(int(out[-1]))
        return bool(text) and text[-1].isalnum()

    @staticmethod
    def _force(row: torch.Tensor, tok: int) -> torch.Tensor:
        keep = row[tok].clone()
        row.fill_(NEG_INF)
        row[tok] = keep if keep > NEG_INF else 0.0
        return row

    # ------------------------------------------------------------------ the processor
    def __call__(self, row: torch.Tensor, seq) -> torch.Tensor:
        out = seq.output_tokens
        self._advance(out)
        st = self.stats
        st.positions += 1
        # a forced tag in progress owns the position
        if self._forcing:
            return self._force(row, self._forcing.pop(0))
        if self.guard_pinned and int(torch.isfinite(row).sum()) <= 1:
            return row                       # an earlier processor already pinned this position (e.g. the think budget)
        single_close = len(self.close) == 1
        # 1. confidence streak (reads only)
        if self.in_think and self.streak > 0 and self.close and self._think_tokens >= self.min_think_tokens:
            p1 = float(torch.softmax(row.float(), -1).max())
            self._run = self._run + 1 if p1 >= self.conf_p else 0
            if self._run >= self.streak:
                self.force_end_thinking = True
        # 2. mid-word defer of the close tag
        mid = self.in_think and self._mid_word(out)
        if mid and single_close:
            row[self.close[0]] = NEG_INF
            st.mid_word_defers += 1
        # 3. armed early end of thinking, at a word boundary
        if self.in_think and self.force_end_thinking and self.close and not mid:
            self.force_end_thinking = False
            self._run = 0
            st.early_think_ends += 1
            self._forcing = list(self.close[1:])
            return self._force(row, self.close[0])
        # 4. after the close tag neither tag may come back
        if self.think_ended:
            hit = False
            if single_close:
                row[self.close[0]] = NEG_INF
                hit = True
            if len(self.open) == 1:
                row[self.open[0]] = NEG_INF
                hit = True
            st.post_close_masks += int(hit)
        # 5. tool-call opener inside thinking / in a detected loop
        if len(self.tool) == 1:
            if self.in_think:
                row[self.tool[0]] = NEG_INF
                st.tool_masks += 1
            elif self.suppress_tool_call:
                row[self.tool[0]] += self.tool_loop_bias
                st.tool_biases += 1
        # 6. one-shot pin to the tool-call opener right after the close tag
        if self._pin_pending and self.think_just_ended and self.tool and not self.tool_opened and not self.in_think:
            self._pin_pending = False
            st.pinned_tool_calls += 1
            self._forcing = list(self.tool[1:])
            return self._force(row, self.tool[0])
        self._pin_pending = self._pin_pending and self.think_just_ended
        # 7. top-1 / top-2 margin (reads only)
        if self.margin and row.numel() >= 2:
            top2 = torch.topk(row.float(), 2).values
            if top2[1] > NEG_INF:
                gap = float(top2[0] - top2[1])             # a difference of logits is a difference of log-probabilities
                st.min_gap = min(st.min_gap, gap)
                st.low_margin += int(gap < self.low_margin)
        return row


def repeated_tool_call(messages: Optional[List[dict]], repeats: int = 3) -> bool:
    """True when the last ``repeats`` assistant turns of a conversation made the identical tool call (name and
    arguments): the signal on which the tool-call opener is biased down for the next turn."""
    calls = []
    for m in messages or []:
        if m.get("role") == "assistant" and m.get("tool_calls"):
            tc = m["tool_calls"][-1]
            fn = tc.get("function", tc)
            calls.append((fn.get("name"), str(fn.get("arguments"))))
        elif m.get("role") == "assistant":
            calls.append(None)
    tail = calls[-repeats:]
    return len(tail) == repeats and tail[0] is not None and all(c == tail[0] for c in tail)
