"""ctypes binding of the sm_100a kernel library (``atlas_b200/_C/libatlas_b200_kernels.so``).

Every wrapper here launches hand-written kernels on the current CUDA stream; nothing falls back to eager
PyTorch.  A missing library raises at load time.  ``launch_count`` counts kernel-launching calls so that
benchmarks can report how many of this library's kernels ran inside a timed region.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional, Tuple

import torch

from ..utils.trace import TRACER as _TRACER
from . import checked

_LIB = None
_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "_C", "libatlas_b200_kernels.so")

launch_count = 0
# When a list: every kernel-launching call appends (name, CUDA event recorded right after the launch); the time between
# consecutive events is the device time of that call plus whatever ran on the stream since the previous one
# (``bench/step_profile.py`` turns it into a per-kernel table).  None = off.
device_marks = None
_status_ptr: Dict[int, int] = {}
_num_sms: Dict[int, int] = {}
_scratch: Dict[Tuple[int, str], torch.Tensor] = {}

FP8 = torch.float8_e4m3fn
_vp, _ll, _i, _f = C.c_void_p, C.c_longlong, C.c_int, C.c_float


class KernelError(RuntimeError):
    pass


def load() -> None:
    global _LIB
    if _LIB is not None:
        return
    if not os.path.exists(LIB_PATH):
        raise KernelError(f"{LIB_PATH} is missing: run `python -m atlas_b200.build` (the GPU path has no eager fallback)")
    lib = C.CDLL(LIB_PATH)
    lib.atlas_status_ptr.restype = C.c_void_p
    lib.atlas_read_status.restype = C.c_ulonglong
    lib.atlas_gemm.argtypes = [_i, _vp, _vp, _vp, _vp, _ll, _ll, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _i, _i, _vp, _vp, _i, _vp, _vp]
    lib.atlas_gemm_gathered.argtypes = lib.atlas_gemm.argtypes + [_vp, _vp, _ll]
    lib.atlas_rmsnorm.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _f, _i, _vp]
    lib.atlas_silu_mul.argtypes = [_vp, _ll, _i, _i, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp]
    lib.atlas_quant_fp8.argtypes = [_vp, _ll, _i, _i, _vp, _ll, _vp, _ll, _vp]
    lib.atlas_rope_kv_write.argtypes = [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                                        _i, _i, _i, _i, _f, _f, _f, _vp]
    lib.atlas_gated_rmsnorm.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _ll, _i, _i, _i, _f, _vp]
    lib.atlas_wht_d128.argtypes = [_vp, _ll, _i, _i, _vp]
    lib.atlas_attn_decode.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _f, _f, _i, _i, _i,
                                      _i, _i, _i, _vp, _vp, _vp, _vp]
    lib.atlas_attn_prefill.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _f, _f, _f, _i,
                                       _i, _i, _i, _i, _vp]
    lib.atlas_attn_prefill_tc.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _f, _f, _f,
                                          _i, _i, _i, _i, _i, _vp, _vp, _vp, _ll, _vp, _ll]
    lib.atlas_argmax.argtypes = [_vp, _ll, _i, _i, _i, _vp, _vp, _vp]
    lib.atlas_sample.argtypes = [_vp, _ll, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]
    lib.atlas_spec_accept.argtypes = [_vp, _vp, _i, _i, _vp, _vp]
    _LIB = lib
    _bind_optional(lib)


def _bind_optional(lib) -> None:
    """Entry points of translation units that may be added later (MoE, GDN, comm)."""
    from . import cuda_ext
    cuda_ext.bind(lib)


def lib():
    load()
    return _LIB


def _dev(t: torch.Tensor) -> int:
    d = t.device.index
    d = torch.cuda.current_device() if d is None else d
    if d not in _status_ptr:
        rc = lib().atlas_init(d)
        if rc != 0:
            raise KernelError(f"atlas_init({d}) failed: {rc}")
        _status_ptr[d] = lib().atlas_status_ptr(d)
        _num_sms[d] = lib().atlas_num_sms(d)
    return d


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if _TRACER.enabled:
        _TRACER.launch(what)
    if device_marks is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        device_marks.append((what, ev))
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def check_status(device: Optional[int] = None, clear: bool = True) -> int:
    """Synchronise and read the device status word (0 = no bounded wait ever gave up)."""
    d = torch.cuda.current_device() if device is None else device
    if d not in _status_ptr:
        return 0
    return int(lib().atlas_read_status(d, 1 if clear else 0))


_scratch_frozen = False


def freeze_scratch() -> None:
    """Called before the first CUDA-graph capture: from here on a scratch buffer is never replaced, because captured
    kernels keep the old address."""
    global _scratch_frozen
    _scratch_frozen = True


def scratch(name: str, nbytes: int, device, zero_new=None) -> torch.Tensor:
    """Per-device persistent scratch.  A buffer grows on demand until the first CUDA graph has been captured; after
    that a request larger than the buffer raises instead of handing captured kernels' memory back to the allocator
    (reserve the worst case up front with :func:`reserve_scratch`)."""
    key = (device.index if device.index is not None else (torch.cuda.current_device() if device.type == "cuda" else -1), name)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None and _scratch_frozen:
            raise KernelError(f"scratch '{name}' holds {buf.numel()} bytes, {nbytes} requested after a CUDA graph was "
                              "captured: reserve the worst case before capturing")
        from ..utils import guards
        alloc = _scratch_alloc or (lambda n, dev: guards.zeros(f"scratch.{name}", (n,), torch.uint8, dev))
        buf = alloc(max(nbytes, 1 << 20), device)
        _scratch[key] = buf
    return buf


_scratch_alloc = None      # tests replace the allocator to exercise the policy without a GPU


def reserve_scratch(name: str, nbytes: int, device) -> torch.Tensor:
    """Make sure ``name`` holds at least ``nbytes`` (call before any graph capture)."""
    return scratch(name, nbytes, device)


def attention_scratch_bytes(batch_sizes, hq: int, hkv: int, d: int, max_seq_len: int, sms: int) -> Tuple[int, int]:
    """Worst case of the split-K decode attention partials over the given batch sizes: (bytes of the partial outputs,
    bytes of the partial (max, sum) pairs)."""
    po = pml = 0
    for b in batch_sizes:
        s = decode_splits(b, hkv, max_seq_len, sms)
        if s > 1:
            po = max(po, b * hq * s * d * 4)
            pml = max(pml, b * hq * s * 2 * 4)
    return po, pml


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _scale_buf(T: int, kb: int, device) -> torch.Tensor:
    """Activation scales, k-group major: logical ``[T, kb]`` with strides ``(1, T_pad)``; rows are padded to a
    multiple of 128 tokens so the GEMM can fetch a tile's 128 scales with one aligned bulk copy."""
    tp = (T + 127) // 128 * 128
    return torch.empty(kb, tp, dtype=torch.float32, device=device)[:, :T].t()


# ----------------------------------------------------------------------------- elementwise
def quant_fp8(x: torch.Tensor, group: int = 128):
    assert group == 128 and x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1
    T, K = x.shape
    _dev(x)
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    s = _scale_buf(T, K // 128, x.device)
    _check(lib().atlas_quant_fp8(x.data_ptr(), x.stride(0), T, K, q.data_ptr(), K, s.data_ptr(), s.stride(1), _stream()),
           "quant_fp8")
    return q, s


def rmsnorm(x, w, eps, residual=None, plus_one=False, quant=False):
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    T, H = x.shape
    _dev(x)
    res_out = torch.empty(T, H, dtype=x.dtype, device=x.device) if residual is not None else None
    y = q = s = None
    if quant:
        q = torch.empty(T, H, dtype=FP8, device=x.device)
        s = _scale_buf(T, H // 128, x.device)
    else:
        y = torch.empty(T, H, dtype=x.dtype, device=x.device)
    _check(lib().atlas_rmsnorm(x.data_ptr(), x.stride(0), _ptr(residual), residual.stride(0) if residual is not None else 0,
                               w.data_ptr(), _ptr(res_out), H, _ptr(y), H, _ptr(q), H, _ptr(s), s.stride(1) if s is not None else 0,
                               T, H, float(eps), 1 if plus_one else 0, _stream()), "rmsnorm")
    if quant:
        return q, s, res_out
    return y, res_out


def silu_mul(gate_up: torch.Tensor, quant=False, live_tiles: Optional[torch.Tensor] = None):
    assert gate_up.dtype == torch.bfloat16 and gate_up.stride(1) == 1
    T, I2 = gate_up.shape
    I = I2 // 2
    _dev(gate_up)
    if quant:
        q = torch.empty(T, I, dtype=FP8, device=gate_up.device)
        s = _scale_buf(T, I // 128, gate_up.device)
        _check(lib().atlas_silu_mul(gate_up.data_ptr(), gate_up.stride(0), T, I, None, 0, q.data_ptr(), I, s.data_ptr(),
                                    s.stride(1), _ptr(live_tiles), _stream()), "silu_mul")
        return q, s
    y = torch.empty(T, I, dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().atlas_silu_mul(gate_up.data_ptr(), gate_up.stride(0), T, I, y.data_ptr(), I, None, 0, None, 0, _ptr(live_tiles), _stream()),
           "silu_mul")
    return y


def gelu_tanh_mul(gate_up: torch.Tensor, quant=False):
    """``gelu_tanh(gate) * up`` of ``[T, 2I]`` (gate | up): bf16, or FP8 with 128-wide group scales."""
    assert gate_up.dtype == torch.bfloat16 and gate_up.stride(1) == 1
    T, I2 = gate_up.shape
    I = I2 // 2
    _dev(gate_up)
    L = lib()
    if not getattr(L, "_gelu_bound", False):
        L.atlas_gelu_tanh_mul.argtypes = [_vp, _ll, _i, _i, _vp, _ll, _vp, _ll, _vp, _ll, _vp]
        L._gelu_bound = True
    if quant:
        q = torch.empty(T, I, dtype=FP8, device=gate_up.device)
        s = _scale_buf(T, I // 128, gate_up.device)
        _check(L.atlas_gelu_tanh_mul(gate_up.data_ptr(), gate_up.stride(0), T, I, None, 0, q.data_ptr(), I, s.data_ptr(),
                                     s.stride(1), _stream()), "gelu_tanh_mul")
        return q, s
    y = torch.empty(T, I, dtype=gate_up.dtype, device=gate_up.device)
    _check(L.atlas_gelu_tanh_mul(gate_up.data_ptr(), gate_up.stride(0), T, I, y.data_ptr(), I, None, 0, None, 0, _stream()),
           "gelu_tanh_mul")
    return y


def gated_rmsnorm(x, z, w, eps):
    T, H, D = x.shape
    _dev(x)
    assert x.stride(2) == 1 and z.stride(2) == 1 and x.stride(1) == D and z.stride(1) == D
    y = torch.empty(T, H, D, dtype=x.dtype, device=x.device)
    _check(lib().atlas_gated_rmsnorm(x.data_ptr(), x.stride(0), z.data_ptr(), z.stride(0), w.data_ptr(), y.data_ptr(),
                                     H * D, T, H, D, float(eps), _stream()), "gated_rmsnorm")
    return y


# ----------------------------------------------------------------------------- GEMM
_GEMM_WS_BYTES = 64 << 20
_FORCE_BLOCK_N = int(os.environ.get("ATLAS_GEMM_BLOCK_N", "0"))
_FORCE_SPLITS = int(os.environ.get("ATLAS_GEMM_SPLITS", "0"))


def gemm_plan(M: int, N: int, K: int, kind: int, sms: int) -> Tuple[int, int]:
    """(block_n, k-splits) for a problem: fill the SMs first with tiles, then with K splits."""
    k_blocks = (K + (128 if kind == 1 else 64) - 1) // (128 if kind == 1 else 64)
    m_tiles = (M + 127) // 128
    if _FORCE_BLOCK_N:
        bn = _FORCE_BLOCK_N
    elif kind == 0 and m_tiles * ((N + 255) // 256) >= 2 * sms and N % 256 == 0:
        bn = 256          # bf16 accumulates in TMEM across K
    elif kind == 1 and m_tiles * ((N + 255) // 256) >= sms and N % 256 == 0:
        bn = 256          # fp8: half the per-k-group buffer handshakes per FLOP and 0.75x the shared-memory fill of 128
    elif m_tiles * ((N + 127) // 128) >= sms:
        bn = 128
    elif kind == 1 and m_tiles == 1 and K >= 8192 and N % 128 == 0:
        bn = 128          # decode rows, long K: fewer, wider tiles and more K splits (128 x 4096 x 14336: 35.5 -> 31.1 us)
    else:
        bn = 64 if N >= 64 * 8 else 64
    tiles = m_tiles * ((N + bn - 1) // bn)
    splits = 1
    if _FORCE_SPLITS:
        splits = _FORCE_SPLITS
    elif tiles * 2 <= sms and k_blocks >= 8:
        splits = max(1, min(sms // tiles, k_blocks // 4, 16))
    while splits > 1 and splits * m_tiles * 128 * ((N + bn - 1) // bn) * bn * 4 > _GEMM_WS_BYTES:
        splits -= 1
    return bn, splits


def _gemm(kind: int, a: torch.Tensor, b: torch.Tensor, a_scale, b_scale, out: Optional[torch.Tensor],
          ready: Optional[tuple] = None) -> torch.Tensor:
    M, K = a.shape
    N = b.shape[0]
    d = _dev(a)
    assert a.stride(1) == 1 and b.stride(1) == 1 and b.shape[1] == K
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    assert out.stride(1) == 1 and out.dtype == torch.bfloat16
    sms = _num_sms[d]
    bn, splits = gemm_plan(M, N, K, kind, sms)
    if ready is not None and M > 128:
        splits = 1                      # prefill-size gathered operands: tiles start as their rows arrive, K stays whole
    ws = cnt = None
    if splits > 1:
        ws = scratch("gemm_ws", _GEMM_WS_BYTES, a.device)
        cnt = scratch("gemm_counters", 1 << 18, a.device)
    sa_m = sa_k = 0
    if kind == 1:
        kb = a_scale.shape[1]
        if a_scale.stride(0) != 1 or a_scale.stride(1) % 4 or a_scale.stride(1) < (M + 127) // 128 * 128 or a_scale.data_ptr() % 16:
            if ready is not None:
                raise KernelError("gathered activation scales must already be in the GEMM's k-group-major layout")
            fixed = _scale_buf(M, kb, a.device)
            fixed.copy_(a_scale)
            a_scale = fixed
        sa_m, sa_k = a_scale.stride(0), a_scale.stride(1)
        assert b_scale.is_contiguous() and b_scale.dtype == torch.float32 and a_scale.dtype == torch.float32
    args = (kind, a.data_ptr(), b.data_ptr(), out.data_ptr(), _ptr(a_scale), sa_m, sa_k, _ptr(b_scale),
            b_scale.shape[1] if b_scale is not None else 0, M, N, K, a.stride(0), b.stride(0),
            out.stride(0), bn, splits, _ptr(ws), _ptr(cnt), sms, _status_ptr[d], _stream())
    if ready is not None:
        # gathered operand: the scales must be read in place (they arrive with the rows), never through a staged copy
        assert a_scale is None or a_scale.data_ptr() % 16 == 0
        _check(lib().atlas_gemm_gathered(*args, ready[0], ready[1], ready[2]), "gemm_gathered")
    else:
        _check(lib().atlas_gemm(*args), "gemm")
    return out


class _Epilogue(C.Structure):
    """Mirror of ``AtlasEpilogue`` (csrc/host_api.h)."""
    _fields_ = [("mode", _i), ("q_out", _vp), ("ldq", _ll), ("s_out", _vp), ("s_ld", _ll), ("residual", _vp), ("ldr", _ll),
                ("norm_w", _vp), ("norm_plus_one", _i), ("ss_out", _vp), ("ss_out_ld", _ll), ("ss_in", _vp),
                ("ss_in_parts", _i), ("ss_in_ld", _ll), ("ss_inv_h", _f), ("ss_eps", _f)]


def fused_block_n(mode: int, M: int, N: int, K: int, sms: int) -> Tuple[int, int]:
    """Tile width and K splits of a fused-epilogue FP8 GEMM: the epilogue needs whole 128-wide quantisation groups
    inside a tile, i.e. 256-wide tiles for the SwiGLU form and 128- or 256-wide tiles for the residual + norm form."""
    bn, _ = gemm_plan(M, N, K, 1, sms)
    if mode == 1:
        bn = 256
    elif mode == 2:
        bn = 256 if (bn == 256 and N % 256 == 0) else 128
    k_blocks = (K + 127) // 128
    m_tiles = (M + 127) // 128
    tiles = m_tiles * ((N // 2) // 128 if mode == 1 else (N + bn - 1) // bn)
    splits = 1
    if _FORCE_SPLITS:
        splits = min(_FORCE_SPLITS, k_blocks)
    elif tiles * 2 <= sms and k_blocks >= 8:
        splits = max(1, min(sms // tiles, k_blocks // 4, 16))
    while splits > 1 and splits * m_tiles * 128 * ((N + bn - 1) // bn) * bn * 4 > _GEMM_WS_BYTES:
        splits -= 1
    return bn, splits


def gemm_fp8_fused(xq, xs, wq, ws, mode: int = 0, out=None, residual=None, norm_w=None, plus_one=False, ss_in=None, ready=None):
    """FP8 block-scaled GEMM with a fused epilogue (``atlas_gemm_fused``).

    mode 0: returns ``out [M, N]`` bf16.  mode 1 (``wq`` = stacked gate and up rows): returns ``(q [M, N/2] fp8, scales)``
    of ``silu(gate) * up``.  mode 2: adds ``residual`` (updated in place), returns ``(q [M, N] fp8, scales, ss)`` where
    ``q`` is the FP8 form of ``residual * norm_w`` and ``ss = (sums [tiles, M_pad], tiles)`` holds the per-row sums of
    squares the consumer needs for the row's 1/rms factor.  ``ss_in = (sums, tiles, H, eps)`` applies such a deferred
    factor of the A operand to the output rows."""
    M, K = xq.shape
    N = wq.shape[0]
    d = _dev(xq)
    sms = _num_sms[d]
    assert xq.dtype == FP8 and wq.dtype == FP8 and xq.stride(1) == 1 and wq.stride(1) == 1
    if xs.stride(0) != 1 or xs.stride(1) % 4 or xs.stride(1) < (M + 127) // 128 * 128 or xs.data_ptr() % 16:
        if ready is not None:
            raise KernelError("gathered activation scales must already be in the GEMM's k-group-major layout")
        fixed = _scale_buf(M, xs.shape[1], xq.device)
        fixed.copy_(xs)
        xs = fixed
    bn, splits = fused_block_n(mode, M, N, K, sms) if mode else gemm_plan(M, N, K, 1, sms)
    if ready is not None and M > 128:
        splits = 1                      # prefill-size gathered operands: tiles start as their rows arrive, K stays whole
    wsp = cnt = None
    if splits > 1:
        wsp = scratch("gemm_ws", _GEMM_WS_BYTES, xq.device)
        cnt = scratch("gemm_counters", 1 << 18, xq.device)
    e = _Epilogue()
    e.mode = mode
    res = None
    if mode == 0:
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
        res = out
    elif mode == 1:
        I = N // 2
        q = torch.empty(M, I, dtype=FP8, device=xq.device)
        sc = _scale_buf(M, I // 128, xq.device)
        e.q_out, e.ldq, e.s_out, e.s_ld = q.data_ptr(), I, sc.data_ptr(), sc.stride(1)
        res = (q, sc)
    else:
        assert residual is not None and residual.dtype == torch.bfloat16 and residual.stride(1) == 1 and residual.shape == (M, N)
        assert norm_w.dtype == torch.bfloat16 and norm_w.is_contiguous()
        q = torch.empty(M, N, dtype=FP8, device=xq.device)
        sc = _scale_buf(M, N // 128, xq.device)
        tiles = N // bn
        ssb = torch.empty(tiles, (M + 127) // 128 * 128, dtype=torch.float32, device=xq.device)
        e.q_out, e.ldq, e.s_out, e.s_ld = q.data_ptr(), N, sc.data_ptr(), sc.stride(1)
        e.residual, e.ldr, e.norm_w, e.norm_plus_one = residual.data_ptr(), residual.stride(0), norm_w.data_ptr(), 1 if plus_one else 0
        e.ss_out, e.ss_out_ld = ssb.data_ptr(), ssb.stride(0)
        res = (q, sc, (ssb, tiles))
    if ss_in is not None:
        sums, parts, H, eps = ss_in
        e.ss_in, e.ss_in_parts, e.ss_in_ld, e.ss_inv_h, e.ss_eps = sums.data_ptr(), parts, sums.stride(0), 1.0 / H, float(eps)
    L = lib()
    if not getattr(L, "_fused_bound", False):
        L.atlas_gemm_fused.argtypes = L.atlas_gemm.argtypes + [C.POINTER(_Epilogue), _vp, _vp, _ll]
        L._fused_bound = True
    rdy = ready if ready is not None else (None, None, 0)
    _check(L.atlas_gemm_fused(1, xq.data_ptr(), wq.data_ptr(), _ptr(out) if mode == 0 else None, xs.data_ptr(), xs.stride(0),
                              xs.stride(1), ws.data_ptr(), ws.shape[1], M, N, K, xq.stride(0), wq.stride(0),
                              out.stride(0) if mode == 0 else 0, bn, splits, _ptr(wsp), _ptr(cnt), sms, _status_ptr[d], _stream(),
                              C.byref(e), rdy[0], rdy[1], rdy[2]), "gemm_fused")
    return res


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out=None) -> torch.Tensor:
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if x.stride(1) != 1 or (x.stride(0) * 2) % 16 or x.data_ptr() % 16:
        x = x.contiguous()
    return _gemm(0, x, w, None, None, out)


def gemm_fp8_block(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, out=None, ready=None) -> torch.Tensor:
    assert xq.dtype == FP8 and wq.dtype == FP8
    return _gemm(1, xq, wq, xs, ws, out, ready)


def gemm_nvfp4(x, packed, bscale, gscale, out=None):
    from . import cuda_ext
    return cuda_ext.gemm_nvfp4(x, packed, bscale, gscale, out)


# ----------------------------------------------------------------------------- KV cache + attention
NVFP4_KV = "nvfp4"        # cache dtype tag: packed e2m1 bytes + e4m3 scales, a uint8 tensor


def is_nvfp4_kv(k_cache: torch.Tensor) -> bool:
    return k_cache.dtype == torch.uint8


def nvfp4_kv_head_dim(k_cache: torch.Tensor) -> int:
    """head_dim of an NVFP4 cache view ``[nb, bs, Hkv, D * 9 / 16]``."""
    return k_cache.shape[3] * 16 // 9


def alloc_kv_cache(num_blocks: int, block_size: int, hkv: int, d: int, dtype, device):
    """Physical layout K ``[nb, Hkv, bs, D]``, V ``[nb, Hkv, D, bs]``; both returned as logical
    ``[nb, bs, Hkv, D]`` views so indexing code is layout-agnostic.

    ``dtype = "nvfp4"``: every (block, kv head) page is ``bs * D * 9 / 16`` bytes, packed e2m1 data followed by e4m3
    scales (one per token and 16 dims; the arrangement inside a page is the kernels' business, see ``paged_attn_kernel``
    in csrc/attention.cu).  The tensors are uint8 views of logical shape ``[nb, bs, Hkv, D * 9 / 16]``: block-level copies
    (prefix cache, host tier) work on them like on any other cache, element indexing does not."""
    from ..utils import guards
    if dtype == NVFP4_KV or dtype == torch.uint8:
        assert d % 16 == 0 and block_size % 16 == 0
        w = d * 9 // 16
        k = guards.zeros("kv.k", (num_blocks, hkv, block_size, w), torch.uint8, device).permute(0, 2, 1, 3)
        v = guards.zeros("kv.v", (num_blocks, hkv, w, block_size), torch.uint8, device).permute(0, 3, 1, 2)
        return k, v
    k = guards.zeros("kv.k", (num_blocks, hkv, block_size, d), dtype, device).permute(0, 2, 1, 3)
    v = guards.zeros("kv.v", (num_blocks, hkv, d, block_size), dtype, device).permute(0, 3, 1, 2)
    return k, v


def _kv_layout_ok(k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    nb, bs, hkv, d = k_cache.shape
    if k_cache.stride() != (hkv * bs * d, d, bs * d, 1) or v_cache.stride() != (hkv * bs * d, 1, d * bs, bs):
        raise KernelError("KV cache is not in the kernel layout (allocate it with ops.cuda.alloc_kv_cache)")
    if k_cache.dtype not in (FP8, torch.bfloat16, torch.uint8):
        raise KernelError("the GPU attention kernels read an FP8 (e4m3), bf16 or NVFP4 KV cache")


def wht_d128(x: torch.Tensor) -> torch.Tensor:
    """In-place orthonormal Walsh-Hadamard rotation of every 128-wide head of ``x [T, H, 128]`` (bf16)."""
    T, H, D = x.shape
    _dev(x)
    if D != 128 or x.dtype != torch.bfloat16 or x.stride(2) != 1 or x.stride(1) != D:
        raise KernelError("wht_d128 takes bf16 rows of 128-wide heads")
    _check(lib().atlas_wht_d128(x.data_ptr(), x.stride(0), T, H, _stream()), "wht_d128")
    return x


def qk_norm_rope_kv_write(q, k, v, positions, rope_cache, rotary_dim, k_cache, v_cache, slot_mapping, k_scale, v_scale,
                          q_norm_w, k_norm_w, eps, norm_plus_one, rotate=False):
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    _dev(q)
    _kv_layout_ok(k_cache, v_cache)
    assert q.stride(2) == 1 and q.stride(1) == D and k.stride(1) == D and v.stride(1) == D
    assert positions.dtype == torch.int32 and slot_mapping.dtype == torch.int32 and rope_cache.dtype == torch.float32
    bs = k_cache.shape[1]
    if is_nvfp4_kv(k_cache) and nvfp4_kv_head_dim(k_cache) != D:
        raise KernelError("NVFP4 KV cache was allocated for a different head_dim")
    kv_mode = (2 if is_nvfp4_kv(k_cache) else (1 if k_cache.dtype == FP8 else 0)) | (8 if rotate else 0)
    if checked.ENABLED:
        checked.kv_write(slot_mapping, positions, k_cache.shape[0], bs, rope_cache.shape[0] if rotary_dim else 0)
    _check(lib().atlas_rope_kv_write(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                                     positions.data_ptr(), rope_cache.data_ptr(), _ptr(q_norm_w), _ptr(k_norm_w),
                                     k_cache.data_ptr(), v_cache.data_ptr(), slot_mapping.data_ptr(), T, Hq, Hkv, D,
                                     rotary_dim, bs, kv_mode, 1 if norm_plus_one else 0, float(eps), float(k_scale),
                                     float(v_scale), _stream()), "rope_kv_write")
    return q


_FORCE_DECODE_SPLITS = int(os.environ.get("ATLAS_DECODE_SPLITS", "0"))


def decode_splits(B: int, hkv: int, max_seq_len: int, sms: int) -> int:
    if _FORCE_DECODE_SPLITS:
        return _FORCE_DECODE_SPLITS
    ctas = B * hkv
    if ctas >= 2 * sms:
        return 1
    pages = (max_seq_len + 15) // 16
    return int(max(1, min((2 * sms + ctas - 1) // ctas, (pages + 7) // 8, 64)))


def paged_attention(q, k_cache, v_cache, batch, scale, k_scale, v_scale, sliding_window):
    T, Hq, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    d = _dev(q)
    _kv_layout_ok(k_cache, v_cache)
    out = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
    bt = batch.block_tables
    window = int(sliding_window or 0)
    nd = batch.num_decodes
    st = _stream()
    if checked.ENABLED:
        checked.paged_read(batch.block_tables, batch.seq_lens, k_cache.shape[0], k_cache.shape[1])
    if k_cache.dtype == torch.bfloat16:
        return _paged_attention_kv16(q, out, k_cache, v_cache, batch, scale, window, d)
    if is_nvfp4_kv(k_cache):
        return _paged_attention_kv16(q, out, k_cache, v_cache, batch, scale, window, d, scales=(float(k_scale), float(v_scale)))
    if nd > 0:
        splits = decode_splits(nd, Hkv, batch.max_seq_len, _num_sms[d])
        po = pml = None
        if splits > 1:
            po = scratch("attn_part_o", nd * Hq * splits * D * 4, q.device)
            pml = scratch("attn_part_ml", nd * Hq * splits * 2 * 4, q.device)
        _check(lib().atlas_attn_decode(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, k_cache.data_ptr(),
                                       v_cache.data_ptr(), bt.data_ptr(), bt.stride(0), batch.seq_lens.data_ptr(),
                                       batch.query_start_loc.data_ptr(), 0, nd, float(scale), float(k_scale),
                                       float(v_scale), Hq, Hkv, D, bs, window, splits, _ptr(po), _ptr(pml), _status_ptr[d], st),
               "attn_decode")
    if batch.num_seqs > nd and _tc_prefill_ok(q, Hq, Hkv, D, bs, window, k_cache):
        # tensor-core (tcgen05) chunk attention: tiles of 128 / G query tokens, all G heads of a kv head per tile
        tdev, n_tiles, _ = _tc_tiles(q, batch, nd, 128 // (Hq // Hkv))
        rc = lib().atlas_attn_prefill_tc(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, k_cache.data_ptr(),
                                         v_cache.data_ptr(), bt.data_ptr(), bt.stride(0), batch.seq_lens.data_ptr(),
                                         batch.query_start_loc.data_ptr(), tdev[0].data_ptr(), tdev[1].data_ptr(), n_tiles,
                                         T, float(scale), float(k_scale), float(v_scale), Hq, Hkv, D, bs, window,
                                         _status_ptr[d], st, None, 0, None, 0)
        if rc != 1:
            _check(rc, "attn_prefill_tc")
            return out
    if batch.num_seqs > nd:
        tiles = getattr(batch, "_attn_tiles", None)
        if tiles is None:
            ts, tq = [], []
            for i in range(nd, batch.num_seqs):
                for q0 in range(0, batch.query_lens_host[i], 16):
                    ts.append(i)
                    tq.append(q0)
            host = torch.tensor([ts, tq], dtype=torch.int32).pin_memory()
            tiles = (host.to(q.device, non_blocking=True), len(ts))
            batch._attn_tiles = tiles
        tdev, n_tiles = tiles
        _check(lib().atlas_attn_prefill(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, k_cache.data_ptr(),
                                        v_cache.data_ptr(), bt.data_ptr(), bt.stride(0), batch.seq_lens.data_ptr(),
                                        batch.query_start_loc.data_ptr(), tdev[0].data_ptr(), tdev[1].data_ptr(),
                                        n_tiles, float(scale), float(k_scale), float(v_scale), Hq, Hkv, D, bs, window,
                                        st), "attn_prefill")
    return out


def paged_attention_q8(q, k_cache, v_cache, batch, scale, k_scale, v_scale, sliding_window):
    """Attention whose kernels write FP8 rows ``[T, Hq * D]`` and one scale per (row, head), the form the output
    projection's FP8 GEMM reads, instead of bf16: decode rows through ``atlas_attn_decode_q8``, prefill chunks through the
    tcgen05 chunk kernel's FP8 epilogue, both into the same buffers for a mixed step.  FP8 cache, head_dim 128; returns
    None when some part of the step is not covered (nothing launched then)."""
    T, Hq, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    if D != 128 or k_cache.dtype != FP8 or T == 0 or batch.num_seqs == 0:
        return None
    nd = batch.num_decodes
    window = int(sliding_window or 0)
    has_chunks = batch.num_seqs > nd
    if has_chunks and (not _tc_prefill_ok(q, Hq, Hkv, D, bs, window, k_cache) or (q.data_ptr() & 15) or (q.stride(0) * 2) % 16):
        return None
    if not has_chunks and nd != T:
        return None
    d = _dev(q)
    _kv_layout_ok(k_cache, v_cache)
    if checked.ENABLED:
        checked.paged_read(batch.block_tables, batch.seq_lens, k_cache.shape[0], k_cache.shape[1])
    L = lib()
    if not getattr(L, "_attn_q8_bound", False):
        L.atlas_attn_decode_q8.argtypes = [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _f, _f, _i,
                                           _i, _i, _i, _i, _vp, _vp, _vp, _vp]
        L._attn_q8_bound = True
    qo = torch.empty(T, Hq * D, dtype=FP8, device=q.device)
    so = _scale_buf(T, Hq, q.device)
    bt = batch.block_tables
    if nd > 0:
        splits = decode_splits(nd, Hkv, batch.max_seq_len, _num_sms[d])
        po = pml = None
        if splits > 1:
            po = scratch("attn_part_o", nd * Hq * splits * D * 4, q.device)
            pml = scratch("attn_part_ml", nd * Hq * splits * 2 * 4, q.device)
        _check(L.atlas_attn_decode_q8(q.data_ptr(), q.stride(0), qo.data_ptr(), Hq * D, so.data_ptr(), so.stride(1),
                                      k_cache.data_ptr(), v_cache.data_ptr(), bt.data_ptr(), bt.stride(0),
                                      batch.seq_lens.data_ptr(), batch.query_start_loc.data_ptr(), 0, nd, float(scale),
                                      float(k_scale), float(v_scale), Hq, Hkv, bs, window, splits, _ptr(po),
                                      _ptr(pml), _status_ptr[d], _stream()), "attn_decode")
    if has_chunks:
        tdev, n_tiles, _ = _tc_tiles(q, batch, nd, 128 // (Hq // Hkv))
        rc = L.atlas_attn_prefill_tc(q.data_ptr(), q.stride(0), None, 0, k_cache.data_ptr(), v_cache.data_ptr(), bt.data_ptr(),
                                     bt.stride(0), batch.seq_lens.data_ptr(), batch.query_start_loc.data_ptr(),
                                     tdev[0].data_ptr(), tdev[1].data_ptr(), n_tiles, T, float(scale), float(k_scale),
                                     float(v_scale), Hq, Hkv, D, bs, window, _status_ptr[d], _stream(), qo.data_ptr(), Hq * D,
                                     so.data_ptr(), so.stride(1))
        if rc == 1:
            raise KernelError("tcgen05 chunk attention refused a shape its eligibility check accepted")
        _check(rc, "attn_prefill_tc")
    return qo, so


def _tc_tiles(q, batch, nd: int, tok: int):
    """(device tensor [2, n] of (sequence, first chunk token) per query tile of ``tok`` tokens, n, tok), cached on the batch."""
    tiles = getattr(batch, "_attn_tiles_tc", None)
    if tiles is None or tiles[2] != tok:
        work = []
        for i in range(nd, batch.num_seqs):
            qlen = batch.query_lens_host[i]
            ctx = batch.seq_lens_host[i] - qlen
            for q0 in range(0, qlen, tok):
                work.append((-(ctx + min(q0 + tok, qlen)), i, q0))        # keys the tile's last row sees
        # tiles with the most keys first: a causal tile costs up to 8x another, and blocks are handed to SMs in index
        # order, so the short ones fill the tail of the launch instead of the long ones making it
        work.sort()
        ts, tq = [w[1] for w in work], [w[2] for w in work]
        host = torch.tensor([ts, tq], dtype=torch.int32).pin_memory()
        tiles = (host.to(q.device, non_blocking=True), len(ts), tok)
        batch._attn_tiles_tc = tiles
    return tiles


def _paged_attention_kv16(q, out, k_cache, v_cache, batch, scale, window, d, scales=None):
    """bf16 KV cache (or, with ``scales = (k_scale, v_scale)``, an NVFP4 one): the general mma.sync kernel serves decode
    rows (split-K + merge) and prefill tiles."""
    T, Hq, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    L = lib()
    fp4 = scales is not None
    if fp4 and not getattr(L, "_kv4_bound", False):
        L.atlas_attn_decode_kv4.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _f, _f, _i, _i, _i, _i, _i,
                                            _i, _vp, _vp, _vp]
        L.atlas_attn_prefill_kv4.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _f, _f, _f, _i, _i, _i,
                                             _i, _i, _vp]
        L._kv4_bound = True
    if fp4 and D not in (128,):
        raise KernelError("the NVFP4 KV cache is implemented for head_dim 128")
    if not getattr(L, "_kv16_bound", False):
        L.atlas_attn_decode_kv16.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _i, _i, _i, _i, _i, _i,
                                             _vp, _vp, _vp]
        L.atlas_attn_prefill_kv16.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _f, _i, _i, _i, _i, _i, _vp]
        L._kv16_bound = True
    bt, st, nd = batch.block_tables, _stream(), batch.num_decodes
    if nd > 0:
        splits = decode_splits(nd, Hkv, batch.max_seq_len, _num_sms[d])
        po = pml = None
        if splits > 1:
            po = scratch("attn_part_o", nd * Hq * splits * D * 4, q.device)
            pml = scratch("attn_part_ml", nd * Hq * splits * 2 * 4, q.device)
        if fp4:
            _check(L.atlas_attn_decode_kv4(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, k_cache.data_ptr(), v_cache.data_ptr(),
                                           bt.data_ptr(), bt.stride(0), batch.seq_lens.data_ptr(), batch.query_start_loc.data_ptr(),
                                           0, nd, float(scale), scales[0], scales[1], Hq, Hkv, D, bs, window, splits, _ptr(po),
                                           _ptr(pml), st), "attn_decode_kv4")
        else:
            _check(L.atlas_attn_decode_kv16(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, k_cache.data_ptr(), v_cache.data_ptr(),
                                            bt.data_ptr(), bt.stride(0), batch.seq_lens.data_ptr(), batch.query_start_loc.data_ptr(),
                                            0, nd, float(scale), Hq, Hkv, D, bs, window, splits, _ptr(po), _ptr(pml), st),
                   "attn_decode_kv16")
    if batch.num_seqs > nd:
        tiles = getattr(batch, "_attn_tiles", None)
        if tiles is None:
            ts, tq = [], []
            for i in range(nd, batch.num_seqs):
                for q0 in range(0, batch.query_lens_host[i], 16):
                    ts.append(i)
                    tq.append(q0)
            host = torch.tensor([ts, tq], dtype=torch.int32).pin_memory()
            tiles = (host.to(q.device, non_blocking=True), len(ts))
            batch._attn_tiles = tiles
        tdev, n_tiles = tiles
        if fp4:
            _check(L.atlas_attn_prefill_kv4(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, k_cache.data_ptr(), v_cache.data_ptr(),
                                            bt.data_ptr(), bt.stride(0), batch.seq_lens.data_ptr(), batch.query_start_loc.data_ptr(),
                                            tdev[0].data_ptr(), tdev[1].data_ptr(), n_tiles, float(scale), scales[0], scales[1], Hq,
                                            Hkv, D, bs, window, st), "attn_prefill_kv4")
        else:
            _check(L.atlas_attn_prefill_kv16(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, k_cache.data_ptr(), v_cache.data_ptr(),
                                             bt.data_ptr(), bt.stride(0), batch.seq_lens.data_ptr(), batch.query_start_loc.data_ptr(),
                                             tdev[0].data_ptr(), tdev[1].data_ptr(), n_tiles, float(scale), Hq, Hkv, D, bs, window, st),
                   "attn_prefill_kv16")
    return out


def lora_bgmv(x: torch.Tensor, slot_of_row: torch.Tensor, adapters: dict, scaling: dict, y: torch.Tensor, col0: int, n: int) -> None:
    """``y[:, col0:col0+n] += scaling_s * B_s (A_s x)`` per row with the row's adapter slot (in place, bf16)."""
    d = _dev(x)
    L = lib()
    if not getattr(L, "_lora_bound", False):
        L.atlas_lora_bgmv.argtypes = [_vp, _ll, _vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i), C.POINTER(_f), _vp, _ll, _i,
                                      _i, _i, _i, _vp]
        L._lora_bound = True
    A, B = (_vp * 8)(), (_vp * 8)()
    rk, sc = (_i * 8)(), (_f * 8)()
    keep = []
    for slot, (a, b) in adapters.items():
        if not (0 < slot < 8):
            continue
        a16, b16 = _bf16_cached(a), _bf16_cached(b)
        keep += [a16, b16]
        A[slot], B[slot], rk[slot], sc[slot] = a16.data_ptr(), b16.data_ptr(), a16.shape[0], float(scaling[slot])
    if x.dtype != torch.bfloat16 or x.stride(1) != 1:
        x = x.bfloat16().contiguous()
    _check(L.atlas_lora_bgmv(x.data_ptr(), x.stride(0), slot_of_row.data_ptr(), A, B, rk, sc, y.data_ptr(), y.stride(0), col0,
                             x.shape[0], x.shape[1], n, _stream()), "lora_bgmv")


_bf16_cache: dict = {}


def _bf16_cached(t: torch.Tensor) -> torch.Tensor:
    hit = _bf16_cache.get(t.data_ptr())
    if hit is None or hit[0] is not t:
        hit = _bf16_cache[t.data_ptr()] = (t, t.to(torch.bfloat16).contiguous())
    return hit[1]


_TC_PREFILL = os.environ.get("ATLAS_ATTN_TC", "1") not in ("0", "false")


def _tc_prefill_ok(q, Hq, Hkv, D, bs, window, k_cache) -> bool:
    return (_TC_PREFILL and D == 128 and bs == 16 and not window and Hq % Hkv == 0 and (Hq // Hkv) in (1, 2, 4, 8)
            and q.dtype == torch.bfloat16 and k_cache.dtype == torch.float8_e4m3fn)


# ----------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, with_value: bool = False):
    """Row-wise argmax (lowest index on ties); ``with_value`` also returns the row maxima as fp32."""
    B, V = logits.shape
    _dev(logits)
    assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
    out = torch.empty(B, dtype=torch.int64, device=logits.device)
    val = torch.empty(B, dtype=torch.float32, device=logits.device) if with_value else None
    _check(lib().atlas_argmax(logits.data_ptr(), logits.stride(0), B, V, 1 if logits.dtype == torch.bfloat16 else 0,
                              out.data_ptr(), _ptr(val), _stream()), "argmax")
    return (out, val) if with_value else out


def sample(logits, temperature, top_k, top_p, min_p, uniform):
    B, V = logits.shape
    _dev(logits)
    if logits.dtype not in (torch.bfloat16, torch.float32):
        logits = logits.float()
    out = torch.empty(B, dtype=torch.int64, device=logits.device)
    _check(lib().atlas_sample(logits.data_ptr(), logits.stride(0), B, V, 1 if logits.dtype == torch.bfloat16 else 0,
                              temperature.float().contiguous().data_ptr(), top_k.to(torch.int32).contiguous().data_ptr(),
                              top_p.float().contiguous().data_ptr(), min_p.float().contiguous().data_ptr(),
                              uniform.float().contiguous().data_ptr(), out.data_ptr(), _stream()), "sample")
    return out


def logit_edits(logits: torch.Tensor, edits: torch.Tensor) -> None:
    """Apply ``edits [n, 6]`` (int32 view of {row, token, add, rep, sub, flags} records) to fp32 ``logits`` in place."""
    B, V = logits.shape
    _dev(logits)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and edits.dtype == torch.int32 and edits.is_contiguous()
    L = lib()
    if not getattr(L, "_edits_bound", False):
        L.atlas_logit_edits.argtypes = [_vp, _ll, _i, _i, _vp, _i, _vp]
        L._edits_bound = True
    _check(L.atlas_logit_edits(logits.data_ptr(), logits.stride(0), B, V, edits.data_ptr(), edits.shape[0], _stream()), "logit_edits")


def spec_accept(draft: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    B, K = draft.shape
    _dev(draft)
    out = torch.empty(B, dtype=torch.int32, device=draft.device)
    _check(lib().atlas_spec_accept(draft.contiguous().data_ptr(), target.contiguous().data_ptr(), B, K, out.data_ptr(),
                                   _stream()), "spec_accept")
    return out


# ----------------------------------------------------------------------------- MoE / GDN (cuda_ext)
def moe_route(logits, top_k, norm_topk, scoring, bias=None, n_group=0, topk_group=0, scale=1.0, hash_table=None, token_ids=None):
    from . import cuda_ext
    return cuda_ext.moe_route(logits, top_k, norm_topk, scoring, bias, n_group, topk_group, scale, hash_table, token_ids)


def moe_forward(x, topk_w, topk_ids, experts, e_lo, pctx, ep_mode):
    from . import cuda_ext
    return cuda_ext.moe_forward(x, topk_w, topk_ids, experts, e_lo, pctx, ep_mode)


def gdn_forward(layer, mixed, a, b, batch, state, commit):
    from . import cuda_ext
    return cuda_ext.gdn_forward(layer, mixed, a, b, batch, state, commit)


def gdn_commit(layer, mixed, a, b, qlens, slots, has_state, state, num_accepted_rows):
    from . import cuda_ext
    return cuda_ext.gdn_commit(layer, mixed, a, b, qlens, slots, has_state, state, num_accepted_rows)


def mamba2_forward(layer, xbc, dt, batch, state, commit):
    from . import cuda_gdn
    return cuda_gdn.mamba2_forward(layer, xbc, dt, batch, state, commit)


def mamba2_commit(layer, xbc, dt, qlens, slots, has_state, state, num_accepted_rows):
    from . import cuda_gdn
    return cuda_gdn.mamba2_commit(layer, xbc, dt, qlens, slots, has_state, state, num_accepted_rows)


def mamba2_gated_norm(y, z, w, group, eps):
    from . import cuda_gdn
    return cuda_gdn.mamba2_gated_norm(y, z, w, group, eps)


def relu_squared(x):
    from . import cuda_gdn
    return cuda_gdn.relu_squared(x)


def sigmoid_gate_mul(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``x *= sigmoid(gate)`` in place, rows of ``n`` bf16 values (``gate`` may be a strided column view)."""
    T, n = x.shape
    _dev(x)
    L = lib()
    if not getattr(L, "_gate_bound", False):
        L.atlas_sigmoid_gate_mul.argtypes = [_vp, _ll, _vp, _ll, _i, _i, _vp]
        L.atlas_shared_expert_blend.argtypes = [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _i, _i, _vp]
        L._gate_bound = True
    _check(L.atlas_sigmoid_gate_mul(x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0), T, n, _stream()), "sigmoid_gate_mul")
    return x


def shared_expert_blend(y: torch.Tensor, s: torch.Tensor, x: torch.Tensor, wg: torch.Tensor) -> torch.Tensor:
    """``y += s * sigmoid(x @ wg^T)`` in place (``wg [1, H]``)."""
    T, H = y.shape
    _dev(y)
    sigmoid_gate_mul  # binds the entry points on first use of either
    L = lib()
    if not getattr(L, "_gate_bound", False):
        L.atlas_sigmoid_gate_mul.argtypes = [_vp, _ll, _vp, _ll, _i, _i, _vp]
        L.atlas_shared_expert_blend.argtypes = [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _i, _i, _vp]
        L._gate_bound = True
    _check(L.atlas_shared_expert_blend(y.data_ptr(), y.stride(0), s.data_ptr(), s.stride(0), x.data_ptr(), x.stride(0),
                                       wg.data_ptr(), T, H, _stream()), "shared_expert_blend")
    return y
