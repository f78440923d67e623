"""Request-level evidence: fingerprints of what a chat request generated, returned in ``usage`` when the request sets
``atlas_evidence: true``, so that a client can check "drafted equals serial", "concurrent equals solo" or "resumed equals
fresh" by comparing two responses instead of reading logs.

* ``atlas_token_sha``: SHA-256 (lowercase hex) of the generated token ids as little-endian ``u32`` in order, reasoning and
  content together, the terminal stop token excluded.
* ``atlas_output_sha256``: SHA-256 of ``SHA-256(content bytes) || SHA-256(reasoning bytes)`` (UTF-8, raw digests, content
  first), so it does not depend on how the text was cut into stream chunks; tool calls do not contribute.
* several choices: the SHA-256 of the per-choice raw digests concatenated in index order; one choice: its own digest.

Compare like with like (two blocking or two streaming requests).  Reference parity:
``crates/spark-server/src/api/evidence.rs`` (field names and digest definitions).
"""
from __future__ import annotations

import hashlib
import struct
from typing import Iterable, List, Sequence


class ChoiceEvidence:
    """Accumulates one choice, delta by delta."""

    def __init__(self, stop_ids: Iterable[int] = ()):
        self.stop_ids = set(int(t) for t in stop_ids)
        self.tokens: List[int] = []
        self._content = hashlib.sha256()
        self._reasoning = hashlib.sha256()

    def add(self, token_ids: Sequence[int] = (), content: str = "", reasoning: str = "") -> None:
        self.tokens.extend(int(t) for t in token_ids)
        if content:
            self._content.update(content.encode("utf-8"))
        if reasoning:
            self._reasoning.update(reasoning.encode("utf-8"))

    def token_digest(self, finish_reason: str = "") -> bytes:
        toks = self.tokens
        if toks and finish_reason == "stop" and toks[-1] in self.stop_ids:
            toks = toks[:-1]
        return hashlib.sha256(struct.pack(f"<{len(toks)}I", *toks)).digest()

    def output_digest(self) -> bytes:
        return hashlib.sha256(self._content.digest() + self._reasoning.digest()).digest()


def combine(digests: Sequence[bytes]) -> str:
    if len(digests) == 1:
        return digests[0].hex()
    return hashlib.sha256(b"".join(digests)).hexdigest()
