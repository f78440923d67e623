"""Quantization formats, restated in plain PyTorch.

These functions define the numerics of every quantized operand the engine
touches and are the oracles the CUDA kernels are tested against:

* FP8 e4m3, one fp32 scale per 128x128 weight tile (``weight_scale_inv``);
  activations get one fp32 scale per token per 128-wide K group.  The GEMM
  accumulates each 128-K group in fp32 and folds ``a_scale * b_scale`` between
  groups (two-level accumulation; reference:
  ``kernels/gb10/common/fp8_gemm_t_blockscaled.cu:15-17``).
* NVFP4: packed E2M1 nibbles, one e4m3 scale per 16 elements, one fp32 global
  scale (reference: ``book/src/deep-dives/nvfp4.md:7-12``,
  ``kernels/gb10/common/quantize_bf16_to_nvfp4.cu``).
"""
from __future__ import annotations

from typing import Tuple

import torch

FP8_MAX = 448.0
E2M1_MAX = 6.0
FP8 = torch.float8_e4m3fn

# magnitudes of the 8 E2M1 codes (sign is bit 3 of the nibble)
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e2m1_lut(device) -> torch.Tensor:
    mags = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=device)
    return torch.cat([mags, -mags])


# ----------------------------------------------------------------------------- FP8 block
def quantize_fp8_block(w: torch.Tensor, block: Tuple[int, int] = (128, 128)) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [N,K]`` -> (fp8 ``[N,K]``, fp32 scale ``[ceil(N/bn), ceil(K/bk)]``) with ``w ~= q * scale``."""
    N, K = w.shape
    bn, bk = block
    nb, kb = (N + bn - 1) // bn, (K + bk - 1) // bk
    wp = torch.zeros(nb * bn, kb * bk, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    tiles = wp.view(nb, bn, kb, bk)
    amax = tiles.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (tiles / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX)
    q = q.reshape(nb * bn, kb * bk)[:N, :K].to(FP8)
    return q.contiguous(), scale.contiguous()


def dequantize_fp8_block(q: torch.Tensor, scale: torch.Tensor, block: Tuple[int, int] = (128, 128)) -> torch.Tensor:
    N, K = q.shape
    bn, bk = block
    s = scale.float().repeat_interleave(bn, 0)[:N].repeat_interleave(bk, 1)[:, :K]
    return q.float() * s


def per_token_group_quant_fp8(x: torch.Tensor, group: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [T,K]`` -> (fp8 ``[T,K]``, fp32 scale ``[T, K/group]``); ``K % group == 0``."""
    T, K = x.shape
    assert K % group == 0, f"K={K} must be a multiple of {group}"
    xg = x.float().view(T, K // group, group)
    amax = xg.abs().amax(-1).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (xg / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(T, K)
    return q, scale


def fp8_block_gemm_ref(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor,
                       block: Tuple[int, int] = (128, 128), out_dtype=torch.bfloat16) -> torch.Tensor:
    """``y[T,N] = sum_g (xq[:,g] @ wq[:,g].T) * xs[:,g] * ws[n/bn, g]`` with fp32 accumulation."""
    T, K = xq.shape
    N = wq.shape[0]
    bn, bk = block
    kb = (K + bk - 1) // bk
    xf, wf = xq.float(), wq.float()
    acc = torch.zeros(T, N, dtype=torch.float32, device=xq.device)
    wsn = ws.float().repeat_interleave(bn, 0)[:N]          # [N, kb]
    for g in range(kb):
        ks = slice(g * bk, min(K, (g + 1) * bk))
        part = xf[:, ks] @ wf[:, ks].t()
        acc += part * xs[:, g].float()[:, None] * wsn[:, g][None, :]
    return acc.to(out_dtype)


# ----------------------------------------------------------------------------- NVFP4
def _round_to_e2m1_code(x: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 code (ties to even mantissa) of ``x`` already divided by its scale."""
    ax = x.abs().clamp(max=E2M1_MAX)
    # decision boundaries between consecutive magnitudes, ties-to-even
    code = torch.zeros_like(ax, dtype=torch.uint8)
    bounds = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
    tie_up = (False, True, False, True, False, True, False)  # at a tie, go up iff upper code is even
    for i, (b, up) in enumerate(zip(bounds, tie_up)):
        code = torch.where((ax > b) | ((ax == b) & up), torch.full_like(code, i + 1), code)
    sign = (x < 0).to(torch.uint8) << 3
    return code | sign


def quantize_nvfp4(w: torch.Tensor, group: int = 16) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``w [N,K]`` -> (packed uint8 ``[N,K/2]`` low nibble first, e4m3 scale ``[N,K/group]``, fp32 global)."""
    N, K = w.shape
    assert K % group == 0 and group % 2 == 0
    wf = w.float()
    amax_t = wf.abs().amax().clamp_min(1e-12)
    gscale = (amax_t / (FP8_MAX * E2M1_MAX)).reshape(1)       # weight_scale_2
    g = wf.view(N, K // group, group)
    bamax = g.abs().amax(-1)
    bs = (bamax / E2M1_MAX / gscale).clamp(max=FP8_MAX).to(FP8)
    bsf = bs.float() * gscale
    bsf = torch.where(bsf == 0, torch.ones_like(bsf), bsf)
    codes = _round_to_e2m1_code(g / bsf[..., None]).view(N, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, bs.contiguous(), gscale.to(torch.float32)


def dequantize_nvfp4(packed: torch.Tensor, bscale: torch.Tensor, gscale: torch.Tensor, group: int = 16) -> torch.Tensor:
    N, K2 = packed.shape
    K = K2 * 2
    lut = _e2m1_lut(packed.device)
    lo = lut[(packed & 0xF).long()]
    hi = lut[(packed >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).view(N, K)
    g = gscale.float().reshape(-1)                       # one global scale, or one per output row (fused projections)
    g = g[0] if g.numel() == 1 else g[:, None]
    s = (bscale.float() * g).repeat_interleave(group, 1)
    return vals * s


def quantize_nvfp4_activations(x: torch.Tensor, gscale: torch.Tensor, group: int = 16):
    """Activation-side NVFP4 (per 16 elements e4m3 scale against a calibrated global scale)."""
    T, K = x.shape
    g = x.float().view(T, K // group, group)
    bs = (g.abs().amax(-1) / E2M1_MAX / gscale).clamp(max=FP8_MAX).to(FP8)
    bsf = bs.float() * gscale
    bsf = torch.where(bsf == 0, torch.ones_like(bsf), bsf)
    codes = _round_to_e2m1_code(g / bsf[..., None]).view(T, K)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous(), bs.contiguous()


# ----------------------------------------------------------------------------- KV cache FP8 (per-tensor scale)
def quant_kv_fp8(x: torch.Tensor, scale: float) -> torch.Tensor:
    return (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)


def f32_to_bf16_rne(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even fp32 -> bf16 (what every kernel epilogue does)."""
    return x.to(torch.bfloat16)


# ----------------------------------------------------------------------------- MXFP4 (OCP microscaling: 32 e2m1 values, e8m0 scale)
def dequantize_mxfp4(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """``blocks [..., K/32, 16]`` uint8 (two e2m1 codes per byte, low nibble first), ``scales [..., K/32]`` uint8 e8m0
    (value ``2 ** (s - 127)``) -> fp32 ``[..., K]``."""
    lut = _e2m1_lut(blocks.device)
    lo, hi = lut[(blocks & 0xF).long()], lut[(blocks >> 4).long()]
    vals = torch.stack([lo, hi], -1).reshape(*blocks.shape[:-1], 32)
    sc = torch.exp2(scales.to(torch.float32) - 127.0)
    return (vals * sc[..., None]).reshape(*blocks.shape[:-2], -1)


def quantize_mxfp4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [N, K]`` -> (blocks ``[N, K/32, 16]`` uint8, scales ``[N, K/32]`` uint8 e8m0): power-of-two scale per 32 values
    chosen so the block maximum fits under 6 (the e2m1 maximum)."""
    N, K = w.shape
    g = w.float().view(N, K // 32, 32)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -126)
    e = torch.ceil(torch.log2(amax / E2M1_MAX)).clamp(-127, 127)
    codes = _round_to_e2m1_code(g / torch.exp2(e)[..., None]).view(N, K // 32, 32)
    blocks = (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()
    return blocks, (e + 127).to(torch.uint8)


def mxfp4_to_nvfp4(blocks: torch.Tensor, scales: torch.Tensor):
    """Re-express MXFP4 ``[N, K/32, 16] + [N, K/32]`` in the NVFP4 layout this engine's kernels read: the codes are the
    same e2m1 values; each 32-block scale becomes two 16-block e4m3 scales against one global power of two.  Exact when
    the scales of the tensor span at most the 17 binades e4m3 holds exactly (2**-9 .. 2**8); returns None otherwise
    (the caller widens to 16 bits instead)."""
    N = blocks.shape[0]
    e = scales.to(torch.int32) - 127
    live = e[scales > 0] if bool((scales > 0).any()) else e
    lo, hi = int(live.min()), int(live.max())
    if hi - lo > 17:
        return None
    shift = hi - 8                                        # the largest scale maps to 2**8
    rel = (e - shift).clamp(-9, 8)
    s16 = torch.exp2(rel.float()).to(FP8)                 # powers of two in range are exact in e4m3
    s16 = torch.where((scales == 0) & (e < lo), torch.zeros_like(s16.float()).to(FP8), s16)
    packed = blocks.reshape(N, -1).contiguous()
    return packed, s16.repeat_interleave(2, dim=-1).contiguous(), torch.tensor([2.0 ** shift], dtype=torch.float32)


# ----------------------------------------------------------------------------- MLX affine group quantisation
def dequantize_mlx(weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group_size: int) -> torch.Tensor:
    """``weight [N, K * bits / 32]`` uint32 (values packed little-endian inside each word), ``scales`` / ``biases``
    ``[N, K / group_size]`` -> fp32 ``[N, K]`` with ``w = q * scale + bias``."""
    N = weight.shape[0]
    per = 32 // bits
    w = weight.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(per, device=weight.device, dtype=torch.int64) * bits
    q = ((w[..., None] >> shifts) & ((1 << bits) - 1)).reshape(N, -1).float()
    K = q.shape[1]
    s = scales.float().repeat_interleave(group_size, 1)[:, :K]
    b = biases.float().repeat_interleave(group_size, 1)[:, :K]
    return q * s + b


def quantize_mlx(w: torch.Tensor, bits: int = 4, group_size: int = 64):
    N, K = w.shape
    g = w.float().view(N, K // group_size, group_size)
    mn, mx = g.amin(-1), g.amax(-1)
    scale = ((mx - mn) / ((1 << bits) - 1)).clamp_min(1e-12)
    q = torch.round((g - mn[..., None]) / scale[..., None]).clamp(0, (1 << bits) - 1).to(torch.int64).view(N, K)
    per = 32 // bits
    shifts = torch.arange(per, dtype=torch.int64) * bits
    packed = (q.view(N, K // per, per) << shifts).sum(-1)
    packed = torch.where(packed >= (1 << 31), packed - (1 << 32), packed).to(torch.int32)
    return packed, scale, mn


# ----------------------------------------------------------------------------- NVFP4 KV cache pages
_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e2m1_to_float(nibbles: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(_E2M1_VALUES + tuple(-v for v in _E2M1_VALUES), dtype=torch.float32, device=nibbles.device)
    return lut[nibbles.long()]


def dequantize_nvfp4_kv(k_cache: torch.Tensor, v_cache: torch.Tensor, head_dim: int):
    """The logical ``[nb, bs, Hkv, D]`` fp32 contents of an NVFP4 KV cache (uint8 views as allocated by
    ``ops.cuda.alloc_kv_cache(..., "nvfp4", ...)``), WITHOUT the tensors' second-level scales.

    Page of K per (block, kv head): ``[bs][D/2]`` packed e2m1 (even dim in the low nibble) then ``[bs][D/16]`` e4m3 scales;
    page of V: ``[D][bs/2]`` packed (even token in the low nibble) then ``[D/16][bs]`` scales.  The oracle of the kernel
    tests; reference parity: ``kernels/gb10/common/reshape_and_cache.cu`` (nvfp4 entry), ``paged_decode_attn_nvfp4.cu``."""
    nb, bs, hkv, w = k_cache.shape
    D = head_dim
    assert w == D * 9 // 16
    kp = k_cache.permute(0, 2, 1, 3).reshape(nb, hkv, bs * w)
    kd = kp[..., :bs * D // 2].reshape(nb, hkv, bs, D // 2)
    ks = kp[..., bs * D // 2:].reshape(nb, hkv, bs, D // 16).contiguous().view(torch.float8_e4m3fn).float()
    kv = torch.stack([_e2m1_to_float(kd & 0xF), _e2m1_to_float(kd >> 4)], -1).reshape(nb, hkv, bs, D)
    K = (kv.view(nb, hkv, bs, D // 16, 16) * ks[..., None]).reshape(nb, hkv, bs, D).permute(0, 2, 1, 3)
    vp = v_cache.permute(0, 2, 3, 1).reshape(nb, hkv, w * bs)
    vd = vp[..., :D * bs // 2].reshape(nb, hkv, D, bs // 2)
    vs = vp[..., D * bs // 2:].reshape(nb, hkv, D // 16, bs).contiguous().view(torch.float8_e4m3fn).float()
    vv = torch.stack([_e2m1_to_float(vd & 0xF), _e2m1_to_float(vd >> 4)], -1).reshape(nb, hkv, D, bs)
    V = (vv.view(nb, hkv, D // 16, 16, bs) * vs[:, :, :, None, :]).reshape(nb, hkv, D, bs).permute(0, 3, 1, 2)
    return K.contiguous(), V.contiguous()
