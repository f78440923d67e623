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


# Row-parallel projection + all-reduce + residual add + norm + FP8 quantisation in ONE kernel (the one-shot fused GEMM with
# the residual / norm epilogue).  Numerically checked by the multi-rank self test, but off by default: the epilogue needs
# 128-wide tiles, and the tile's last CTA then runs split-K reduction, peer exchange and the row epilogue back to back,
# which measured slower at 2 GPUs (5.30 against 4.86 ms per decode step of the 8B shape) than 64-wide tiles plus a separate
# norm kernel.  ATLAS_TP_FUSED_NORM=1 switches it on.
TP_FUSED_NORM = os.environ.get("ATLAS_TP_FUSED_NORM", "0") == "1"


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
        return self.all_reduce(ops.linear(act, w))

    def row_parallel_residual_norm(self, act, w, residual: torch.Tensor, norm_w: torch.Tensor, eps: float, plus_one: bool):
        """Row-parallel projection whose kernel also sums over the TP group, adds the sum to ``residual`` (in place) and
        emits the FP8 activations of ``residual * norm_w`` with the 1/rms factor deferred (``Act.row_ss``).  Returns
        ``(Act, residual)`` or None when this backend / shape has no such kernel (nothing was launched)."""
        from .. import ops
        if not TP_FUSED_NORM:
            return None
        if not (self.tp_size > 1 and self.comm is not None and hasattr(self.comm, "gemm_allreduce")):
            return None
        if not ops.residual_norm_fusable(residual, w):
            return None
        a = act if isinstance(act, ops.Act) else ops.Act(x=act)
        r = self.comm.gemm_allreduce(a, w, epilogue=(residual, norm_w, plus_one))
        if r is None:
            return None
        q, s, (sums, parts) = r
        return ops.Act(q=q, s=s, dtype=residual.dtype, row_ss=(sums, parts, w.weight.shape[0], eps)), residual

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
