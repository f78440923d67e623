"""NVFP4 x NVFP4 (W4A4) GEMM on the block-scaled tensor-core path and its activation quantiser (``csrc/gemm_fp4.cu``).

Scale factors travel in the 128 x 4 atom order the tensor core reads (see the kernel header); ``sf_atoms`` puts a plain
``[rows, K/16]`` e4m3 matrix (checkpoint layout) into that order once, at load time, and ``sf_from_atoms`` undoes it for
tests.

Reference parity: ``kernels/gb10/qwen3.6-27b/nvfp4/w4a4_gemm.cu``, ``kernels/gb10/common/quantize_nvfp4.cu``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import cuda as K

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float


def _lib():
    L = K.lib()
    if not getattr(L, "_fp4_bound", False):
        L.atlas_quant_nvfp4.argtypes = [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp]
        L.atlas_gemm_nvfp4_w4a4.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _f, _vp, _ll, _i, _i, _i, _i, _vp, _vp]
        L._fp4_bound = True
    return L


def atom_bytes(rows: int, k: int) -> int:
    return ((rows + 127) // 128) * ((k + 63) // 64) * 512


def sf_atoms(scale: torch.Tensor) -> torch.Tensor:
    """``scale [rows, K/16]`` (e4m3 or uint8) -> flat uint8 buffer in atom order, zero padded."""
    s = scale.view(torch.uint8)
    rows, groups = s.shape
    rb, kg = (rows + 127) // 128, (groups + 3) // 4
    pad = torch.zeros(rb * 128, kg * 4, dtype=torch.uint8, device=s.device)
    pad[:rows, :groups] = s
    # [rb, 4 (row/32), 32 (row%32), kg, 4] -> [rb, kg, 32, 4, 4]
    return pad.view(rb, 4, 32, kg, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)


def sf_from_atoms(atoms: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    rb, kg = (rows + 127) // 128, (k + 63) // 64
    s = atoms.view(rb, kg, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(rb * 128, kg * 4)
    return s[:rows, :k // 16].contiguous()


def quant_nvfp4(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """bf16 ``x [M, K]`` -> (packed e2m1 ``[M, K/2]`` uint8, scale-factor atoms, per-row second-level scale ``[M]``)."""
    M, Kd = x.shape
    K._dev(x)
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and Kd % 32 == 0
    q = torch.empty(M, Kd // 2, dtype=torch.uint8, device=x.device)
    sf = torch.zeros(atom_bytes(M, Kd), dtype=torch.uint8, device=x.device)
    rs = torch.empty(M, dtype=torch.float32, device=x.device)
    K._check(_lib().atlas_quant_nvfp4(x.data_ptr(), x.stride(0), M, Kd, q.data_ptr(), sf.data_ptr(), rs.data_ptr(), K._stream()),
             "quant_nvfp4")
    return q, sf, rs


def gemm_w4a4(xq: torch.Tensor, xsf: torch.Tensor, row_scale: Optional[torch.Tensor], wq: torch.Tensor, wsf: torch.Tensor,
              col_scale: Optional[torch.Tensor], alpha: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out [M, N]`` bf16 from packed e2m1 operands ``xq [M, K/2]``, ``wq [N, K/2]`` and their scale-factor atoms."""
    M, K2 = xq.shape
    N = wq.shape[0]
    d = K._dev(xq)
    assert wq.shape[1] == K2 and xq.is_contiguous() and wq.is_contiguous()
    assert xsf.numel() >= atom_bytes(M, 2 * K2) and wsf.numel() >= atom_bytes(N, 2 * K2)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
    K._check(_lib().atlas_gemm_nvfp4_w4a4(xq.data_ptr(), xsf.data_ptr(), K._ptr(row_scale), wq.data_ptr(), wsf.data_ptr(),
                                          K._ptr(col_scale), float(alpha), out.data_ptr(), out.stride(0), M, N, 2 * K2,
                                          K._num_sms[d], K._status_ptr[d], K._stream()), "gemm_nvfp4_w4a4")
    return out


def dequant(q: torch.Tensor, sf: torch.Tensor, outer: Optional[torch.Tensor], rows: int, k: int) -> torch.Tensor:
    """fp32 matrix a (packed, atoms, per-row scale) triple stands for."""
    from .. import quant as Q
    s = sf_from_atoms(sf, rows, k).view(torch.float8_e4m3fn)
    g = torch.ones(1, device=q.device) if outer is None else outer
    return Q.dequantize_nvfp4(q, s, g)


def linear_w4a4(x: torch.Tensor, w, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ W^T`` for an NVFP4 ``LinearWeight`` with the activations quantised to NVFP4 on the fly (per-row second-level
    scale).  The weight's scale factors are put into atom order once and cached on the weight object."""
    cache = getattr(w, "_w4a4", None)
    if cache is None:
        N = w.weight.shape[0]
        g = w.gscale.float().reshape(-1)
        col = (g.expand(N) if g.numel() == 1 else g).contiguous()
        cache = w._w4a4 = (sf_atoms(w.scale), col)
    if x.dtype != torch.bfloat16:
        x = x.bfloat16()
    if x.stride(-1) != 1:
        x = x.contiguous()
    xq, xsf, xrs = quant_nvfp4(x)
    return gemm_w4a4(xq, xsf, xrs, w.weight, cache[0], cache[1], out=out)
