"""Output sanitisation: what keeps template markers, tool-call markup and runaway repetition out of the text a client
sees.

Four pieces, used by both the streaming and the blocking path:

* :func:`guarded_stops`: chat-template control markers spelled out as text (``<|im_end|>``, a new ``<|im_start|>user``
  header, ...) mean "this turn is over"; they join the request's stop strings, so the streaming hold-back logic cuts
  the output in front of a complete one even across chunk boundaries.
* :class:`ContentSanitizer`: a streaming filter for the CONTENT channel (after reasoning splitting and tool parsing).
  Complete tool-call markup tags that survive the parser are removed (exact tags like ``</tool_call>`` and
  attribute-style openers like ``<function=name>`` through their ``>``), everything between an envelope opener and its
  closer is suppressed, stray ``</think>`` markers are dropped, and the longest suffix that could still grow into a
  marker is held back until the next chunk decides.  ``flush`` at the end of the stream drops what is still held when
  it is an unfinished tag or when a suppressed envelope never closed.
* :func:`strip_orphan_tool_markup` / :func:`scrub_think_markers` / :func:`scrub_tool_tags`: the same rules for a
  complete string (blocking responses).
* :class:`StreamGuards`: a cap on tool calls per response and a repetition watchdog over the visible text (the last
  non-trivial line seen four times in the recent window, compared with collapsed whitespace, or a phrase of 30+
  characters recurring four times).

``--no-output-sanitizer`` turns all of it off.

Reference behaviour replaced: ``crates/spark-server/src/api/sanitizer.rs`` (streaming content sanitiser with marker
hold-back), ``scrub.rs`` (complete-tag scrubbing), ``strip.rs`` (thinking markers, orphan tool markup),
``stream_guards.rs`` (tool-call cap, loop watchdog, end-of-stream flush).
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass, field
from typing import Iterable, List, Sequence, Tuple

LEAK_MARKERS = (
    "<|im_end|>", "<|im_start|>", "<|endoftext|>", "<|eot_id|>", "<|start_header_id|>", "<|end_header_id|>",
    "<|begin_of_text|>", "<|end_of_text|>", "<|end|>", "<|user|>", "<|assistant|>", "<|system|>", "[INST]", "[/INST]",
    "<end_of_turn>", "<start_of_turn>",
)


def guarded_stops(user_stops: Iterable[str], enabled: bool = True) -> List[str]:
    """The request's stop strings plus the leak markers (no duplicates, user strings first)."""
    stops = [x for x in user_stops if x]
    if enabled:
        stops += [m for m in LEAK_MARKERS if m not in stops]
    return stops


@dataclass(frozen=True)
class ToolMarkers:
    """Markup a tool dialect uses.  ``envelope_open`` / ``envelope_close`` bracket a call whose body must never reach
    the content channel; ``exact`` are complete tags to drop wherever they appear; ``attr_open`` are openers that carry
    an attribute and end at the next ``>`` (``<function=get_weather>``)."""
    envelope_open: Tuple[str, ...] = ("<tool_call>", "<|tool_call_begin|>", "<|tool_calls_section_begin|>", "[TOOL_CALLS]")
    envelope_close: Tuple[str, ...] = ("</tool_call>", "<|tool_call_end|>", "<|tool_calls_section_end|>")
    exact: Tuple[str, ...] = ("</tool_call>", "<tool_call>", "</function>", "</parameter>", "<|tool_call_end|>",
                              "<|tool_call_begin|>", "<|tool_calls_section_begin|>", "<|tool_calls_section_end|>", "</_call>")
    attr_open: Tuple[str, ...] = ("<function=", "<parameter=")
    think: Tuple[str, ...] = ("</think>", "<think>")

    @property
    def all(self) -> Tuple[str, ...]:
        return tuple(dict.fromkeys(self.envelope_open + self.envelope_close + self.exact + self.attr_open + self.think))


DEFAULT_MARKERS = ToolMarkers()


def marker_prefix_hold(buf: str, markers: Sequence[str]) -> int:
    """Length of the longest suffix of ``buf`` that is a proper prefix of some marker: the only characters that could
    still combine with a later chunk into a marker."""
    top = min(len(buf), max((len(m) for m in markers), default=1) - 1)
    for k in range(top, 0, -1):
        tail = buf[-k:]
        if any(m.startswith(tail) for m in markers):
            return k
    return 0


def scrub_tool_tags(text: str, markers: ToolMarkers = DEFAULT_MARKERS) -> str:
    """Remove every COMPLETE tool-markup tag; an attribute opener without its ``>`` ends the scan (the rest is a tag that
    was still being formed and is dropped)."""
    out = []
    i, n = 0, len(text)
    while i < n:
        if text[i] not in "<[":
            j = i + 1
            while j < n and text[j] not in "<[":
                j += 1
            out.append(text[i:j])
            i = j
            continue
        hit = next((m for m in markers.exact if text.startswith(m, i)), None)
        if hit is not None:
            i += len(hit)
            continue
        attr = next((m for m in markers.attr_open if text.startswith(m, i)), None)
        if attr is not None:
            end = text.find(">", i)
            if end < 0:
                break
            i = end + 1
            continue
        out.append(text[i])
        i += 1
    return "".join(out)


def scrub_think_markers(text: str, markers: ToolMarkers = DEFAULT_MARKERS) -> str:
    """Drop every thinking marker that survived the reasoning split and the whitespace right after it."""
    for m in markers.think:
        while m in text:
            a = text.index(m)
            text = text[:a] + text[a + len(m):].lstrip()
    return text


def strip_orphan_tool_markup(text: str, markers: ToolMarkers = DEFAULT_MARKERS) -> str:
    """Cut the content at the first tool-call opener (used when NO tool call was parsed: whatever follows the opener is
    an orphan block, not prose)."""
    cuts = [text.find(m) for m in markers.envelope_open + markers.attr_open if m in text]
    return text[:min(cuts)].rstrip() if cuts else text


class ContentSanitizer:
    """Streaming form of the rules above.  ``feed(chunk)`` returns what may be shown now."""

    def __init__(self, markers: ToolMarkers = DEFAULT_MARKERS):
        self.m = markers
        self.buf = ""
        self.suppressing = False           # inside an envelope whose closer has not arrived
        self.dropped = 0

    def feed(self, chunk: str) -> str:
        self.buf += chunk
        out = []
        while self.buf:
            if self.suppressing:
                ends = [(self.buf.find(c), c) for c in self.m.envelope_close if c in self.buf]
                if not ends:
                    keep = marker_prefix_hold(self.buf, self.m.envelope_close)
                    self.dropped += len(self.buf) - keep
                    self.buf = self.buf[len(self.buf) - keep:] if keep else ""
                    break
                pos, c = min(ends)
                self.dropped += pos + len(c)
                self.buf = self.buf[pos + len(c):]
                self.suppressing = False
                continue
            # earliest complete marker in the buffer
            first = None
            for mk in self.m.all:
                p = self.buf.find(mk)
                if p >= 0 and (first is None or p < first[0] or (p == first[0] and len(mk) > len(first[1]))):
                    first = (p, mk)
            if first is None:
                keep = marker_prefix_hold(self.buf, self.m.all)
                out.append(self.buf[:len(self.buf) - keep] if keep else self.buf)
                self.buf = self.buf[len(self.buf) - keep:] if keep else ""
                break
            p, mk = first
            out.append(self.buf[:p])
            rest = self.buf[p + len(mk):]
            if mk in self.m.envelope_open:
                self.suppressing = True
                self.buf = rest
            elif mk in self.m.attr_open:
                end = rest.find(">")
                if end < 0:
                    self.buf = self.buf[p:]              # the opener's end has not arrived: hold it whole
                    break
                self.buf = rest[end + 1:]
            elif mk in self.m.think:
                self.buf = rest.lstrip()
            else:
                self.buf = rest
            self.dropped += len(mk)
        return "".join(out)

    def flush(self) -> str:
        """End of stream: what is still held is shown unless it is an unfinished tag or sits inside an envelope."""
        held, self.buf = self.buf, ""
        if self.suppressing or not held:
            self.dropped += len(held)
            return ""
        if any(held.startswith(a) for a in self.m.attr_open) or marker_prefix_hold(held, self.m.all) == len(held):
            self.dropped += len(held)
            return ""
        return held


_WS = re.compile(r"\s+")


@dataclass
class StreamGuards:
    """Per-response guards evaluated on the visible text as it grows."""
    max_tool_calls: int = field(default_factory=lambda: int(os.environ.get("ATLAS_MAX_TOOL_CALLS_PER_RESPONSE", "12")))
    window: int = 10_240
    repeats: int = 4
    min_line: int = 12
    min_phrase: int = 30
    tool_calls: int = 0
    text: str = ""
    tripped: str = ""

    def on_tool_call(self, n: int = 1) -> bool:
        """True once the response has produced more tool calls than the cap."""
        self.tool_calls += n
        if self.tool_calls > self.max_tool_calls and not self.tripped:
            self.tripped = "tool_call_cap"
        return bool(self.tripped)

    def on_text(self, chunk: str) -> bool:
        """True when the text has started to loop."""
        if self.tripped or not chunk:
            return bool(self.tripped)
        self.text = (self.text + chunk)[-self.window:]
        if "\n" in chunk:
            lines = [_WS.sub(" ", l).strip() for l in self.text.split("\n")]
            done = [l for l in lines[:-1] if len(l) >= self.min_line]
            if done and done.count(done[-1]) >= self.repeats:
                self.tripped = "repeated_line"
                return True
        tail = self.text[-self.min_phrase:]
        if len(tail) == self.min_phrase and len(set(tail)) > 4 and self.text.count(tail) >= self.repeats:
            self.tripped = "repeated_phrase"
        return bool(self.tripped)
