"""Checked mode of the kernel bindings (``ATLAS_CHECKED=1``): every index a kernel is about to trust is validated on
the device first, and a violation raises :class:`KernelError` naming the tensor and the offending value BEFORE the
launch, so a bad index becomes an error message instead of a write into someone else's memory.  It costs a
synchronisation per call and is meant for tests and for reproducing a suspected overrun, not for serving.

The kernels' own device-side guards (bounded waits, capacity checks of the all-to-all and the expert alignment) are
always on and report through the status word; this mode covers what they take on trust: cache slots, block tables,
positions, token and expert ids.

Reference parity: ``crates/spark-runtime/src/cuda_backend/gpu_impl.rs:356`` (``debug_sync_kernels``: synchronise and
check after every launch), capacity guards of ``crates/spark-comm/src/recv_buffer.rs``.
"""
from __future__ import annotations

import os

import torch

ENABLED = os.environ.get("ATLAS_CHECKED", "0") == "1"


class BoundsViolation(RuntimeError):
    pass


def _fail(what: str, detail: str):
    raise BoundsViolation(f"checked mode: {what}: {detail}")


def index_range(what: str, t: torch.Tensor, lo: int, hi: int) -> None:
    """Every element of ``t`` in ``[lo, hi)``."""
    if t is None or t.numel() == 0:
        return
    mn, mx = int(t.min()), int(t.max())
    if mn < lo or mx >= hi:
        _fail(what, f"values span [{mn}, {mx}], allowed [{lo}, {hi})")


def kv_write(slot_mapping: torch.Tensor, positions: torch.Tensor, num_blocks: int, block_size: int, rope_rows: int) -> None:
    index_range("slot_mapping", slot_mapping, -1, num_blocks * block_size)
    if rope_rows:
        index_range("positions", positions, 0, rope_rows)
    live = slot_mapping[slot_mapping >= 0]
    if live.numel() and torch.unique(live).numel() != live.numel():
        _fail("slot_mapping", "two rows of one step write the same cache slot")


def paged_read(block_tables: torch.Tensor, seq_lens: torch.Tensor, num_blocks: int, block_size: int) -> None:
    if seq_lens.numel() == 0:
        return
    need = (seq_lens.to(torch.int64) + block_size - 1) // block_size
    if int(need.max()) > block_tables.shape[1]:
        _fail("block_tables", f"a sequence of {int(seq_lens.max())} tokens needs {int(need.max())} blocks, the table has "
                              f"{block_tables.shape[1]} columns")
    cols = torch.arange(block_tables.shape[1], device=block_tables.device)[None, :]
    used = block_tables[:need.shape[0]][cols < need[:, None]]
    index_range("block_tables (entries covered by seq_lens)", used, 0, num_blocks)


def finite(what: str, t: torch.Tensor) -> None:
    if t.is_floating_point() and t.numel() and not bool(torch.isfinite(t.float()).all()):
        _fail(what, "contains inf or nan")
