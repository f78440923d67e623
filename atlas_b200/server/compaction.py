"""Progressive context compaction: make an over-long chat fit the context window instead of rejecting it.

Applied only when the rendered prompt does not leave ``reserve`` tokens of room, in stages that lose the least first;
after each stage the chat is rendered and counted again:

1. long tool results (role ``tool``), oldest first, are cut to their head and tail around an elision marker;
2. long assistant / user turns older than the last ``keep_recent`` messages get the same treatment;
3. the oldest non-system messages are dropped (a tool result goes with the assistant turn that called it), and one
   system note says how many messages were left out.

System messages and the last ``keep_recent`` messages are never dropped.  Returns the new message list and a report
(stage reached, messages elided / dropped), which the server exposes in the response's usage details.
Reference behaviour replaced: ``crates/spark-server/src/api/compact.rs`` (progressive compaction before the context
length check).
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, List, Tuple

MARK = "\n[... {n} characters elided ...]\n"


def _text_of(msg: dict) -> str:
    c = msg.get("content")
    if isinstance(c, str):
        return c
    if isinstance(c, list):
        return "".join(p.get("text", "") for p in c if isinstance(p, dict))
    return ""


def _set_text(msg: dict, text: str) -> None:
    msg["content"] = text


def _elide(text: str, keep: int) -> str:
    if len(text) <= keep + 64:
        return text
    head = keep * 2 // 3
    tail = keep - head
    return text[:head] + MARK.format(n=len(text) - keep) + text[len(text) - tail:]


def compact_messages(messages: List[dict], count_tokens: Callable[[List[dict]], int], budget: int, keep_recent: int = 4,
                     elide_to: int = 1200) -> Tuple[List[dict], Dict[str, int]]:
    msgs = copy.deepcopy(messages)
    report = {"stage": 0, "elided": 0, "dropped": 0, "tokens_before": count_tokens(msgs)}
    if report["tokens_before"] <= budget:
        report["tokens_after"] = report["tokens_before"]
        return msgs, report
    protected = max(0, len(msgs) - keep_recent)

    def fits() -> bool:
        return count_tokens(msgs) <= budget

    # stage 1 and 2: elide long bodies, tool results first, oldest first
    for stage, roles in ((1, ("tool",)), (2, ("assistant", "user"))):
        report["stage"] = stage
        for i in range(protected):
            m = msgs[i]
            if m.get("role") in roles:
                t = _text_of(m)
                cut = _elide(t, elide_to)
                if cut != t:
                    _set_text(m, cut)
                    report["elided"] += 1
                    if fits():
                        report["tokens_after"] = count_tokens(msgs)
                        return msgs, report
    # stage 3: drop oldest non-system messages; the note that replaces them counts against the budget too
    report["stage"] = 3

    def with_note(ms: List[dict]) -> List[dict]:
        if not report["dropped"]:
            return ms
        note = {"role": "system", "content": f"[{report['dropped']} earlier messages were left out to fit the context window]"}
        pos = next((i for i, m in enumerate(ms) if m.get("role") != "system"), len(ms))
        return ms[:pos] + [note] + ms[pos:]

    while True:
        protected = max(0, len(msgs) - keep_recent)
        idx = next((i for i in range(protected) if msgs[i].get("role") != "system"), None)
        if idx is None:
            break
        n = 1
        if msgs[idx].get("role") == "assistant" and msgs[idx].get("tool_calls"):
            while idx + n < protected and msgs[idx + n].get("role") == "tool":
                n += 1
        del msgs[idx:idx + n]
        report["dropped"] += n
        if count_tokens(with_note(msgs)) <= budget:
            break
    msgs = with_note(msgs)
    report["tokens_after"] = count_tokens(msgs)
    return msgs, report
