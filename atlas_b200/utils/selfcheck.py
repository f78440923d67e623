"""Boot-time kernel self-test (``serve --check-kernels``, ``doctor``): each hot kernel on one small case against the
PyTorch restatement of the same op; raises on a mismatch or a non-zero device status word.

Reference parity: ``--check-kernels`` / kernel audit at boot (``crates/spark-runtime/src/kernel_audit.rs``,
``crates/spark-model/src/preflight.rs``).
"""
from __future__ import annotations

from typing import Dict

import torch


def _rel_rms(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.float()
    return float((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt().clamp_min(1e-12))


def kernel_selftest(device="cuda") -> Dict[str, float]:
    from .. import quant as Q
    from ..ops import cuda as K
    from ..ops import reference as ref
    K.load()
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(7)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev)
    out: Dict[str, float] = {}

    a, b = (rnd(192, 512) * 0.5).bfloat16(), (rnd(384, 512) * 0.5).bfloat16()
    out["gemm_bf16"] = _rel_rms(K.gemm_bf16(a, b), a.float() @ b.float().t())

    x, w = rnd(96, 1024).bfloat16(), rnd(512, 1024) * 0.05
    wq, ws = Q.quantize_fp8_block(w)
    xq, xs = K.quant_fp8(x)
    out["gemm_fp8_block"] = _rel_rms(K.gemm_fp8_block(xq, xs, wq, ws),
                                     Q.fp8_block_gemm_ref(xq, xs.contiguous(), wq, ws, out_dtype=torch.float32))

    h, wn = rnd(64, 1024).bfloat16(), (1 + 0.1 * rnd(1024)).bfloat16()
    y, _ = K.rmsnorm(h, wn, 1e-6, None, False, quant=False)
    yr, _ = ref.rmsnorm(h, wn, 1e-6, None, False)
    out["rmsnorm"] = _rel_rms(y, yr)

    logits = rnd(32, 4096)
    ids = K.argmax(logits)
    out["argmax"] = float((ids.long() != ref.argmax_first(logits).long()).sum())

    torch.cuda.synchronize(dev)
    st = K.check_status()
    bounds = {"gemm_bf16": 6e-3, "gemm_fp8_block": 5e-3, "rmsnorm": 1e-2, "argmax": 0.5}
    bad = {k: v for k, v in out.items() if not (v <= bounds[k])}
    if st or bad:
        raise RuntimeError(f"kernel self-test failed: status word {st:#x}, out of bounds {bad}")
    return out
