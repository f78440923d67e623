"""Checkpoint directory reader: safetensors shards (+index), lazy tensor access, quantised-tensor assembly.

Reads go through ``safetensors.safe_open`` (mmap).  With ``ATLAS_FAST_LOAD=1`` whole shards are streamed by the native
pipelined O_DIRECT reader (``csrc/runtime/direct_io.cpp``) into pinned host memory and tensors are zero-copy views.

Reference parity: ``crates/spark-runtime/src/weights/loader.rs`` (``WeightStore``), ``fast_weights/*`` (O_DIRECT
pipelined loader), ``spark-model/src/weight_map/nvfp4_detect.rs``.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Optional

import torch

from .. import quant as Q
from .qtensor import QTensor


class Checkpoint:
    def __init__(self, path: str):
        self.path = path
        self._where: Dict[str, str] = {}
        self._open: Dict[str, object] = {}
        self._shards: Dict[str, Dict[str, torch.Tensor]] = {}
        self._fast = os.environ.get("ATLAS_FAST_LOAD", "0") not in ("0", "", "false")
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self._where = dict(json.load(f)["weight_map"])
        else:
            from safetensors import safe_open
            for fn in sorted(os.listdir(path)):
                if fn.endswith(".safetensors"):
                    with safe_open(os.path.join(path, fn), framework="pt") as f:
                        for k in f.keys():
                            self._where[k] = fn
        if not self._where:
            raise FileNotFoundError(f"no safetensors weights under {path}")
        self.mlx_group_size = 0
        cfg = os.path.join(path, "config.json")
        if os.path.exists(cfg):
            with open(cfg) as f:
                q = (json.load(f).get("quantization") or {})
            self.mlx_group_size = int(q.get("group_size", 0) or 0)

    def keys(self) -> Iterable[str]:
        return self._where.keys()

    def has(self, name: str) -> bool:
        return name in self._where

    def _file(self, fn: str):
        f = self._open.get(fn)
        if f is None:
            from safetensors import safe_open
            f = safe_open(os.path.join(self.path, fn), framework="pt")
            self._open[fn] = f
        return f

    def get(self, name: str) -> torch.Tensor:
        if self._fast:
            return self._fast_file(self._where[name])[name]
        return self._file(self._where[name]).get_tensor(name)

    # ------------------------------------------------------------------ fast path: whole shard through direct I/O
    _DT = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F8_E4M3": torch.float8_e4m3fn,
           "F8_E5M2": torch.float8_e5m2, "U8": torch.uint8, "I8": torch.int8, "I32": torch.int32, "I64": torch.int64,
           "F64": torch.float64, "BOOL": torch.bool, "I16": torch.int16}

    def _fast_file(self, fn: str) -> Dict[str, torch.Tensor]:
        """Reads the shard once with the native pipelined O_DIRECT reader into one (pinned, when CUDA is present) host
        buffer and hands out zero-copy views; the buffer lives as long as any view does."""
        cached = self._shards.get(fn)
        if cached is not None:
            return cached
        import struct

        from .. import runtime_native as N
        path = os.path.join(self.path, fn)
        size = os.path.getsize(path)
        buf = torch.empty(size, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
        got = N.read_file_into(path, 0, size, buf.data_ptr(), threads=int(os.environ.get("ATLAS_LOAD_THREADS", "8")))
        if got != size:
            raise IOError(f"{path}: short read ({got} of {size} bytes)")
        hlen = struct.unpack("<Q", bytes(buf[:8].tolist()))[0]
        header = json.loads(bytes(buf[8:8 + hlen].numpy().tobytes()).decode())
        base = 8 + hlen
        out: Dict[str, torch.Tensor] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            lo, hi = meta["data_offsets"]
            dt = self._DT[meta["dtype"]]
            raw = buf[base + lo:base + hi]
            out[name] = raw.view(dt).view(meta["shape"]) if hi > lo else torch.empty(meta["shape"], dtype=dt)
        self._shards[fn] = out
        return out

    def maybe(self, name: str) -> Optional[torch.Tensor]:
        return self.get(name) if name in self._where else None

    # ------------------------------------------------------------------ quantised linear weights
    def linear(self, prefix: str) -> QTensor:
        """``prefix`` without ``.weight``.  Recognises FP8 block scales (``weight_scale_inv``), ModelOpt NVFP4
        (``weight`` uint8 + ``weight_scale`` e4m3 + ``weight_scale_2``) and compressed-tensors NVFP4
        (``weight_packed`` + ``weight_scale`` + ``weight_global_scale``)."""
        w = self.maybe(prefix + ".weight")
        # MXFP4 (32-value e2m1 blocks with e8m0 scales): "<prefix>.weight_blocks" / "<prefix>_blocks" + "..._scales"
        for b, sc in ((prefix + ".weight_blocks", prefix + ".weight_scales"), (prefix + "_blocks", prefix + "_scales")):
            if w is None and self.has(b) and self.has(sc):
                blocks, scales = self.get(b).view(torch.uint8), self.get(sc).view(torch.uint8)
                if blocks.dim() == 3:
                    conv = Q.mxfp4_to_nvfp4(blocks, scales)
                    if conv is not None:                 # same e2m1 codes, scales re-expressed: runs on the NVFP4 kernels
                        return QTensor("nvfp4", conv[0], conv[1], conv[2])
                return QTensor("dense", Q.dequantize_mxfp4(blocks, scales).to(torch.bfloat16))
        # MLX affine quantisation: uint32-packed ``weight`` + ``scales`` + ``biases``
        if w is not None and w.dtype in (torch.uint32, torch.int32) and self.has(prefix + ".scales") and self.has(prefix + ".biases"):
            sc, bi = self.get(prefix + ".scales"), self.get(prefix + ".biases")
            group = self.mlx_group_size or 64
            bits = w.shape[1] * 32 // (sc.shape[1] * group)
            return QTensor("dense", Q.dequantize_mlx(w.view(torch.int32), sc, bi, bits, group).to(sc.dtype))
        if w is None and self.has(prefix + ".weight_packed"):
            packed = self.get(prefix + ".weight_packed")
            g = self.get(prefix + ".weight_global_scale").float().reshape(-1)
            # compressed-tensors stores the reciprocal convention: value = e2m1 * scale / global
            return QTensor("nvfp4", packed.view(torch.uint8), self.get(prefix + ".weight_scale").view(torch.float8_e4m3fn),
                           (1.0 / g).reshape(1))
        if w is None:
            raise KeyError(prefix + ".weight")
        if w.dtype == torch.float8_e4m3fn:
            s = self.maybe(prefix + ".weight_scale_inv")
            if s is None:
                s = self.maybe(prefix + ".weight_scale")
            if s is None:
                raise KeyError(f"{prefix}: fp8 weight without a scale tensor")
            s = s.float()
            if s.dim() < 2:      # per-tensor scale -> broadcast to the block grid
                n, k = w.shape
                s = s.reshape(1, 1).expand((n + 127) // 128, (k + 127) // 128).contiguous()
            return QTensor("fp8_block", w, s)
        if w.dtype == torch.uint8 and self.has(prefix + ".weight_scale_2"):
            return QTensor("nvfp4", w, self.get(prefix + ".weight_scale").view(torch.float8_e4m3fn),
                           self.get(prefix + ".weight_scale_2").float().reshape(1))
        return QTensor("dense", w)

    def close(self) -> None:
        self._open.clear()
        self._shards.clear()
