"""Shared layer plumbing: parallel context, weight construction and TP slicing.

TP slicing happens on the high-precision tensor *before* quantization, so every rank quantizes its
own shard (reference: ``crates/spark-model/src/tp_shard.rs:37-120``).
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..ops import LinearWeight


# row-parallel projections of at least this many rows overlap their all-reduce with the next chunk's GEMM
OVERLAP_MIN_ROWS = int(os.environ.get("ATLAS_TP_OVERLAP_MIN_ROWS", "2048"))
# 1 = off.  Measured on 2 x B200 (8192-token prefill steps, 8B model): 73.8 ms with 1 chunk, 75.7 ms with 2, 74.2 ms with
# 4: the persistent GEMM holds every SM, so the reduction of chunk i only gets going when the GEMM of chunk i+1 drains.
OVERLAP_CHUNKS = int(os.environ.get("ATLAS_TP_OVERLAP_CHUNKS", "1"))


@dataclass
class ParallelCtx:
    tp_rank: int = 0
    tp_size: int = 1
    ep_rank: int = 0
    ep_size: int = 1
    comm: Any = None        # parallel.comm.CommBackend over the TP group
    ep_comm: Any = None     # CommBackend over the EP group (may alias ``comm``)

    @property
    def is_tp(self) -> bool:
        return self.tp_size > 1

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1 and self.comm is not None:
            return self.comm.all_reduce(t)
        return t

    def row_parallel_linear(self, act, w) -> torch.Tensor:
        """Row-parallel projection: GEMM on this rank's K-shard, summed over the TP group.  With a peer-memory
        backend the reduction runs inside the GEMM kernel; otherwise GEMM then all-reduce."""
        from .. import ops
        if self.tp_size > 1 and self.comm is not None and hasattr(self.comm, "gemm_allreduce"):
            a = act if isinstance(act, ops.Act) else ops.Act(x=act)
            probe = a.x if a.x is not None else a.q
            if ops.on_gpu(probe):
                y = self.comm.gemm_allreduce(a, w)
                if y is not None:
                    return y
                y = self._row_parallel_overlapped(a, w)
                if y is not None:
                    return y
        return self.all_reduce(ops.linear(act, w))

    def _row_parallel_overlapped(self, a, w) -> Optional[torch.Tensor]:
        """Prefill-size row-parallel projection: the rows are cut into chunks, each chunk's all-reduce is started
        asynchronously as soon as its GEMM is queued, and the next chunk's GEMM runs on the compute stream meanwhile,
        so only the last chunk's reduction is exposed.  Returns None when the shape or the backend does not qualify."""
        from .. import ops
        rows = (a.q if a.q is not None else a.x).shape[0]
        start = getattr(self.comm, "all_reduce_async", None)
        if start is None or OVERLAP_CHUNKS <= 1 or rows < OVERLAP_MIN_ROWS or w.bias is not None or torch.cuda.is_current_stream_capturing():
            return None
        chunks = OVERLAP_CHUNKS
        step = ((rows + chunks - 1) // chunks + 127) // 128 * 128
        y = torch.empty(rows, w.out_features, dtype=a.out_dtype,
                        device=(a.q if a.q is not None else a.x).device)
        pending = []
        for lo in range(0, rows, step):
            hi = min(rows, lo + step)
            part = ops.Act(x=None if a.x is None else a.x[lo:hi], q=None if a.q is None else a.q[lo:hi],
                           s=None if a.s is None else a.s[lo:hi], dtype=a.dtype)
            ops.linear(part, w, out=y[lo:hi])
            pending.append(start(y[lo:hi]))
        for work in pending:
            work.wait()
        return y

    def ep_all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        c = self.ep_comm if self.ep_comm is not None else self.comm
        if self.ep_size > 1 and c is not None:
            return c.all_reduce(t)
        return t


def shard_rows(w: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    """Column-parallel slice (output features)."""
    if size == 1:
        return w
    n = w.shape[0]
    assert n % size == 0, f"rows {n} not divisible by tp {size}"
    s = n // size
    return w[rank * s:(rank + 1) * s]


def shard_cols(w: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    """Row-parallel slice (input features)."""
    if size == 1:
        return w
    k = w.shape[1]
    assert k % size == 0, f"cols {k} not divisible by tp {size}"
    s = k // size
    return w[:, rank * s:(rank + 1) * s]


def randn_weight(gen: torch.Generator, n: int, k: int, std: float, dtype, device) -> torch.Tensor:
    """N(0, std) weight drawn on the generator's device, moved to ``device``."""
    w = torch.randn(n, k, generator=gen, dtype=torch.float32, device=gen.device) * std
    return w.to(device=device, dtype=dtype)


def make_weight(w: torch.Tensor, kind: str, bias: Optional[torch.Tensor] = None) -> LinearWeight:
    """Wrap (and quantize, if asked) a high-precision ``[N,K]`` tensor."""
    n, k = w.shape
    if kind == "fp8_block" and (k % 128 != 0):
        kind = "dense"
    if kind == "nvfp4" and (k % 16 != 0):
        kind = "dense"
    return LinearWeight.from_dense(w, kind, bias)
