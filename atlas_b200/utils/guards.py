"""Red-zone guard bands, an allocation ledger and KV block poisoning: the race / overrun detectors that stand in for a
memory sanitizer.

``GuardedAllocator.alloc`` places every buffer between two bands of a fixed byte pattern inside one larger uint8
allocation; ``scan`` re-reads the bands and reports every buffer whose neighbourhood was written (a kernel that ran
past either end of its buffer).  The ledger lists what was allocated, by whom and how large.  ``poison_block`` fills a
KV block with a pattern that decodes to huge values, so a kernel that reads a block it was not given shows up as
garbage output in the determinism gates instead of passing by luck on stale data; ``zero_block`` is its inverse.

Enabled for the kernel library's own large buffers (paged KV pools, scratch areas) with ``ATLAS_REDZONES=1``; the GPU
test tier switches it on and scans after every test.

Reference parity: ``crates/spark-runtime/src/cuda_backend.rs:157-330`` (``poison_redzones`` / ``scan_redzones``),
``cuda_backend/alloc_ledger.rs``, ``kv_cache/paged_impl.rs:96-129`` (``poison_block`` / ``zero_block``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

CANARY = 0xA5
ZONE_BYTES = 512
POISON_BYTE = 0x7E          # e4m3 0x7E = 448 (largest finite), bf16 0x7E7E = 5.3e37: unmistakable in any output


def enabled() -> bool:
    return os.environ.get("ATLAS_REDZONES", "0") == "1"


@dataclass
class _Entry:
    name: str
    raw: torch.Tensor            # uint8 [zone | payload (padded to 256) | zone]
    payload_bytes: int
    shape: Tuple[int, ...]
    dtype: torch.dtype


@dataclass
class Violation:
    name: str
    side: str                    # "below" | "above"
    offset: int                  # first damaged byte, counted from the band's start
    value: int


class GuardedAllocator:
    def __init__(self, zone_bytes: int = ZONE_BYTES):
        self.zone = zone_bytes
        self.entries: List[_Entry] = []

    def alloc(self, name: str, shape: Sequence[int], dtype: torch.dtype, device, fill: Optional[float] = 0.0) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        padded = (nbytes + 255) // 256 * 256
        raw = torch.full((self.zone + padded + self.zone,), CANARY, dtype=torch.uint8, device=device)
        payload = raw[self.zone:self.zone + nbytes]
        if fill is not None:
            payload.zero_()
        self.entries.append(_Entry(name, raw, nbytes, tuple(int(d) for d in shape), dtype))
        return payload.view(dtype).view(*shape)

    def scan(self) -> List[Violation]:
        bad: List[Violation] = []
        for e in self.entries:
            tail0 = self.zone + e.payload_bytes
            for side, band in (("below", e.raw[:self.zone]), ("above", e.raw[tail0:])):
                hit = (band != CANARY).nonzero()
                if hit.numel():
                    off = int(hit[0])
                    bad.append(Violation(e.name, side, off, int(band[off])))
        return bad

    def repair(self) -> None:
        """Restore the bands (after a reported violation, so that later scans report new damage only)."""
        for e in self.entries:
            e.raw[:self.zone] = CANARY
            e.raw[self.zone + e.payload_bytes:] = CANARY

    def ledger(self) -> List[Dict[str, object]]:
        return [{"name": e.name, "bytes": e.payload_bytes, "shape": e.shape, "dtype": str(e.dtype), "device": str(e.raw.device)}
                for e in self.entries]

    def release(self, name_prefix: str = "") -> int:
        keep = [e for e in self.entries if not e.name.startswith(name_prefix)] if name_prefix else []
        dropped = len(self.entries) - len(keep)
        self.entries = keep
        return dropped


GLOBAL = GuardedAllocator()


def zeros(name: str, shape: Sequence[int], dtype: torch.dtype, device) -> torch.Tensor:
    """``torch.zeros`` with guard bands when red zones are enabled."""
    if enabled():
        return GLOBAL.alloc(name, shape, dtype, device)
    return torch.zeros(*shape, dtype=dtype, device=device)


def _block_bytes(t: torch.Tensor, block: int) -> torch.Tensor:
    """Byte view of one block of a paged pool (logical ``[blocks, ...]`` view of any physical layout)."""
    b = t[block]
    return b.view(torch.uint8) if b.is_contiguous() else b


def poison_block(kv: Tuple[torch.Tensor, torch.Tensor], block: int) -> None:
    for t in kv:
        b = t[block]
        if b.element_size() == 1:
            b.view(torch.uint8).fill_(POISON_BYTE)
        else:
            b.fill_(torch.finfo(b.dtype).max if b.dtype.is_floating_point else 0x7E7E)


def zero_block(kv: Tuple[torch.Tensor, torch.Tensor], block: int) -> None:
    for t in kv:
        b = t[block]
        (b.view(torch.uint8) if b.element_size() == 1 else b).zero_()
