"""Row choice for a reduced-vocabulary draft head.

A draft head that scores ``N < vocab`` rows of the language-model head reads ``N / vocab`` of its bytes per draft step.
A draft can only be a token the head holds, and a miss rejects that draft and every later one of its chain, so which
rows the head holds decides the acceptance rate: the first ``N`` ids (``"id"``) or the ``N`` most frequent tokens of a
recorded table (``"freq"``), with forced ids (end-of-sequence, added tokens) always kept.  Every draft is verified by
the full head, so the emitted tokens do not depend on the choice.

Reference parity: ``crates/spark-model/src/layers/mtp_head/vocab_rank.rs`` (row selection, forced tokens, coverage),
``vocab_recorder.rs`` (counting served tokens into a table).
"""
from __future__ import annotations

import json
from collections import Counter
from typing import Iterable, List, Optional, Sequence


def select_rows(rows: int, vocab: int, ranked_ids: Optional[Sequence[int]] = None, forced: Iterable[int] = ()) -> List[int]:
    """Token id of every head row, ascending (so a tie between two rows resolves to the lower token id, as the full head
    does).  ``ranked_ids``: token ids from most to least frequent; ids it does not list follow in id order."""
    rows = max(1, min(int(rows), int(vocab)))
    keep: List[int] = []
    seen = set()

    def take(t) -> None:
        t = int(t)
        if 0 <= t < vocab and t not in seen and len(keep) < rows:
            seen.add(t)
            keep.append(t)
    for t in forced:
        take(t)
    for t in (ranked_ids or ()):
        take(t)
    t = 0
    while len(keep) < rows:
        take(t)
        t += 1
    return sorted(keep)


def coverage(row_ids: Sequence[int], tokens: Iterable[int]) -> float:
    """Fraction of ``tokens`` a head with these rows could have proposed."""
    have = set(int(t) for t in row_ids)
    n = hit = 0
    for t in tokens:
        n += 1
        hit += int(t) in have
    return hit / n if n else 1.0


def load_ranked_ids(path: str) -> List[int]:
    """A table written by :class:`VocabRecorder` (``{"ids": [...], "counts": [...]}``) or a bare JSON list of ids."""
    with open(path) as f:
        d = json.load(f)
    return [int(t) for t in (d["ids"] if isinstance(d, dict) else d)]


class VocabRecorder:
    """Counts the tokens an engine emits; ``save`` writes them ranked for ``select_rows``."""

    def __init__(self):
        self.counts: Counter = Counter()

    def add(self, tokens: Iterable[int]) -> None:
        self.counts.update(int(t) for t in tokens)

    def ranked(self) -> List[int]:
        return [t for t, _ in sorted(self.counts.items(), key=lambda kv: (-kv[1], kv[0]))]

    def save(self, path: str) -> None:
        ids = self.ranked()
        with open(path, "w") as f:
            json.dump({"ids": ids, "counts": [self.counts[t] for t in ids]}, f)
