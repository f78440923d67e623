"""QTensor: a checkpoint tensor that may already be quantised, with the slicing operations tensor parallelism needs.

FP8 block-scaled tensors carry ``scale [ceil(N/128), ceil(K/128)]``; row / column slices must fall on 128
boundaries to keep the scale grid valid (they do for head-, expert- and 128-multiple FFN shards).  A slice that does
not is served by dequantise -> slice -> requantise.  NVFP4 tensors carry per-row-per-16 scales, so any row slice and
16-aligned column slices are exact.

Reference parity: ``crates/spark-model/src/tp_shard/quant_shard.rs``, ``quant_format/{fp8_blockscaled,modelopt,
compressed_tensors}.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .. import quant as Q
from ..ops import LinearWeight


@dataclass
class QTensor:
    kind: str                               # dense | fp8_block | nvfp4
    weight: torch.Tensor
    scale: Optional[torch.Tensor] = None
    gscale: Optional[torch.Tensor] = None

    @property
    def shape(self) -> Tuple[int, int]:
        n, k = self.weight.shape
        return (n, k * 2) if self.kind == "nvfp4" else (n, k)

    def dequant(self) -> torch.Tensor:
        if self.kind == "dense":
            return self.weight
        if self.kind == "fp8_block":
            return Q.dequantize_fp8_block(self.weight, self.scale)
        return Q.dequantize_nvfp4(self.weight, self.scale, self.gscale)

    def rows(self, lo: int, hi: int) -> "QTensor":
        if self.kind == "dense":
            return QTensor("dense", self.weight[lo:hi])
        if self.kind == "nvfp4":
            g = self.gscale if self.gscale.numel() == 1 else self.gscale.reshape(-1)[lo:hi]
            return QTensor("nvfp4", self.weight[lo:hi], self.scale[lo:hi], g)
        n = self.weight.shape[0]
        if lo % 128 == 0 and (hi % 128 == 0 or hi == n):
            return QTensor("fp8_block", self.weight[lo:hi], self.scale[lo // 128:(hi + 127) // 128])
        if (lo // 128) == ((hi - 1) // 128):        # inside one scale block row
            return QTensor("fp8_block", self.weight[lo:hi], self.scale[lo // 128:lo // 128 + 1])
        return QTensor("dense", self.dequant()[lo:hi])

    def cols(self, lo: int, hi: int) -> "QTensor":
        if self.kind == "dense":
            return QTensor("dense", self.weight[:, lo:hi])
        if self.kind == "nvfp4":
            if lo % 16 == 0 and hi % 16 == 0:
                return QTensor("nvfp4", self.weight[:, lo // 2:hi // 2], self.scale[:, lo // 16:hi // 16], self.gscale)
            return QTensor("dense", self.dequant()[:, lo:hi])
        k = self.weight.shape[1]
        if lo % 128 == 0 and (hi % 128 == 0 or hi == k):
            return QTensor("fp8_block", self.weight[:, lo:hi], self.scale[:, lo // 128:(hi + 127) // 128])
        return QTensor("dense", self.dequant()[:, lo:hi])

    def to(self, device) -> "QTensor":
        mv = lambda t: None if t is None else t.to(device)
        return QTensor(self.kind, mv(self.weight), mv(self.scale), mv(self.gscale))


def as_q(t) -> QTensor:
    return t if isinstance(t, QTensor) else QTensor("dense", t)


def cat_rows(parts: Sequence[QTensor]) -> QTensor:
    """Concatenate along rows (fused QKV / gate|up).  Mixed kinds, or FP8 parts whose row count is not a multiple of
    128 (other than a single-block part), are dequantised."""
    parts = [as_q(p) for p in parts]
    kinds = {p.kind for p in parts}
    if kinds == {"dense"}:
        return QTensor("dense", torch.cat([p.weight for p in parts], 0))
    if kinds == {"fp8_block"} and all(p.weight.shape[0] % 128 == 0 for p in parts[:-1]):
        return QTensor("fp8_block", torch.cat([p.weight for p in parts], 0), torch.cat([p.scale for p in parts], 0))
    if kinds == {"nvfp4"}:
        g = parts[0].gscale
        if all(p.gscale.numel() == 1 and torch.equal(p.gscale, g) for p in parts):
            gs = g
        else:       # parts quantised against different global scales: keep one scale per output row
            gs = torch.cat([p.gscale.float().reshape(-1).expand(p.weight.shape[0]) for p in parts])
        return QTensor("nvfp4", torch.cat([p.weight for p in parts], 0), torch.cat([p.scale for p in parts], 0), gs)
    return QTensor("dense", torch.cat([p.dequant().float() for p in parts], 0))


def to_linear(q: QTensor, want_kind: str, dtype: torch.dtype, bias=None) -> LinearWeight:
    """Final conversion: keep a checkpoint's quantisation as is; quantise high-precision tensors when the model
    configuration asks for it."""
    if q.kind == "fp8_block":
        return LinearWeight("fp8_block", q.weight.contiguous(), q.scale.float().contiguous(), bias=bias)
    if q.kind == "nvfp4":
        return LinearWeight("nvfp4", q.weight.contiguous(), q.scale.contiguous(), q.gscale.float().reshape(-1).contiguous(), bias=bias)
    w = q.weight
    n, k = w.shape
    if want_kind == "fp8_block" and k % 128 == 0:
        return LinearWeight.from_dense(w.float(), "fp8_block", bias)
    if want_kind == "nvfp4" and k % 16 == 0:
        return LinearWeight.from_dense(w.float(), "nvfp4", bias)
    return LinearWeight("dense", w.to(dtype).contiguous(), bias=bias)
