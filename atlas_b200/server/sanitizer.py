"""Output guard against chat-template markers that leak into visible text.

A model whose tokenizer does not carry a template's control tokens as specials (or a fine-tune that learned to spell them
out) can emit ``<|im_end|>``, ``<|eot_id|>``, a new ``<|im_start|>user`` header and so on as ordinary text and then keep
talking to itself.  Every such marker means "this turn is over", so the guard treats them as additional stop strings:
the streaming path already holds back text that could be the beginning of a stop string and cuts the output in front
of a complete one, which gives the marker the same treatment across chunk boundaries.  ``--no-output-sanitizer`` turns
it off.

Reference behaviour replaced: ``crates/spark-server/src/api/sanitizer.rs``, ``stream_guards.rs``, ``strip.rs`` (marker
stripping on the streamed text); the content scrubbing rules of ``scrub.rs`` are not reproduced.
"""
from __future__ import annotations

from typing import Iterable, List

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
