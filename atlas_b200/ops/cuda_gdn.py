"""Binding of the Gated-DeltaNet kernels (``csrc/gdn.cu``)."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from . import cuda as K

_vp, _ll, _i = C.c_void_p, C.c_longlong, C.c_int
_bound = False
USE_CHUNKED = True          # tests switch this off to compare the two kernels
CHUNK_MIN_ROWS = 32


def _lib():
    global _bound
    lib = K.lib()
    if not _bound:
        lib.atlas_gdn_conv.argtypes = [_vp, _ll, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _vp]
        lib.atlas_gdn_conv_state.argtypes = [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp]
        lib.atlas_gdn_recurrent.argtypes = [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp,
                                            _vp, _i, _i, _i, _i, _i, _i, _i, _vp]
        lib.atlas_gdn_chunked.argtypes = [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _i,
                                          _i, _i, _i, _i, _i, _i, _vp]
        _bound = True
    return lib


class _Meta:
    """Device-side per-step sequence metadata shared by all GDN layers of one forward pass."""

    def __init__(self, qlens: List[int], slots: List[int], has_state: List[bool], device, snapshot_plan=None,
                 limit: Optional[List[int]] = None):
        B = len(qlens)
        qsl = [0]
        seq_of = []
        for i, n in enumerate(qlens):
            qsl.append(qsl[-1] + n)
            seq_of.extend([i] * n)
        snaps = max((len(v) for v in (snapshot_plan or {}).values()), default=0)
        rows = [0] * (B * max(1, snaps))
        dsts = [0] * (B * max(1, snaps))
        for i, lst in (snapshot_plan or {}).items():
            for s, (r, d) in enumerate(lst):
                rows[i * snaps + s], dsts[i * snaps + s] = r, d
        ints = torch.tensor(qsl + seq_of + slots + rows + dsts + (limit or []), dtype=torch.int32).pin_memory()
        dev = ints.to(device, non_blocking=True)
        o = 0
        self.qsl = dev[o:o + B + 1]; o += B + 1
        self.seq_of = dev[o:o + len(seq_of)]; o += len(seq_of)
        self.slots = dev[o:o + B]; o += B
        self.snap_rows = dev[o:o + len(rows)]; o += len(rows)
        self.snap_slots = dev[o:o + len(dsts)]; o += len(dsts)
        self.limit = dev[o:o + B] if limit is not None else None
        self.has = torch.tensor([1 if h else 0 for h in has_state], dtype=torch.uint8).pin_memory().to(device, non_blocking=True)
        self.B, self.T, self.snaps = B, len(seq_of), snaps
        # the chunked (64-token, tensor-core) kernel takes prefill-sized steps (a snapshot row just ends a chunk early)
        self.chunk_ok = limit is None and max(qlens, default=0) >= CHUNK_MIN_ROWS


def _run(layer, mixed, a, b, meta: _Meta, state, commit: bool):
    lib, st = _lib(), K._stream()
    K._dev(mixed)
    T, Cc = mixed.shape
    y = torch.empty(T, Cc, dtype=torch.bfloat16, device=mixed.device)
    out = torch.empty(T, layer.hv * layer.dv, dtype=torch.bfloat16, device=mixed.device)
    conv, h = state["conv"], state["h"]
    assert conv.dtype == torch.bfloat16 and h.dtype == torch.float32 and conv.is_contiguous() and h.is_contiguous()
    cw = layer.conv_w if layer.conv_w.dtype == torch.bfloat16 else layer.conv_w.bfloat16()
    K._check(lib.atlas_gdn_conv(mixed.data_ptr(), mixed.stride(0), cw.data_ptr(), Cc, layer.W, conv.data_ptr(),
                                meta.seq_of.data_ptr(), meta.qsl.data_ptr(), meta.slots.data_ptr(), meta.has.data_ptr(),
                                y.data_ptr(), Cc, T, st), "gdn_conv")
    rc = 1
    if USE_CHUNKED and meta.chunk_ok and commit and layer.dk == 128 and layer.dv == 128:
        rc = lib.atlas_gdn_chunked(y.data_ptr(), Cc, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                                   layer.A_log.data_ptr(), layer.dt_bias.data_ptr(), h.data_ptr(), out.data_ptr(),
                                   layer.hv * layer.dv, meta.qsl.data_ptr(), meta.slots.data_ptr(), meta.has.data_ptr(),
                                   meta.snap_rows.data_ptr(), meta.snap_slots.data_ptr(), meta.snaps, meta.B, layer.hk,
                                   layer.hv, layer.dk, layer.dv, 1, st)
        if rc != 1:
            K._check(rc, "gdn_chunked")
    if rc == 1:
      K._check(lib.atlas_gdn_recurrent(y.data_ptr(), Cc, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                                       layer.A_log.data_ptr(), layer.dt_bias.data_ptr(), h.data_ptr(), out.data_ptr(),
                                       layer.hv * layer.dv, meta.qsl.data_ptr(), meta.slots.data_ptr(), meta.has.data_ptr(),
                                       K._ptr(meta.limit), meta.snap_rows.data_ptr(), meta.snap_slots.data_ptr(), meta.snaps,
                                       meta.B, layer.hk, layer.hv, layer.dk, layer.dv, 1 if commit else 0, st), "gdn_recurrent")
    if commit:
        K._check(lib.atlas_gdn_conv_state(mixed.data_ptr(), mixed.stride(0), Cc, layer.W, conv.data_ptr(), meta.qsl.data_ptr(),
                                          meta.slots.data_ptr(), meta.has.data_ptr(), K._ptr(meta.limit),
                                          meta.snap_rows.data_ptr(), meta.snap_slots.data_ptr(), meta.snaps, meta.B, st),
                 "gdn_conv_state")
    return out


def gdn_forward(layer, mixed, a, b, batch, state, commit):
    meta = getattr(batch, "_gdn_meta", None)
    if meta is None:
        meta = _Meta(batch.query_lens_host, batch.state_slots_host, batch.has_state_host, mixed.device, batch.snapshot_plan)
        batch._gdn_meta = meta
    o = _run(layer, mixed, a, b, meta, state, commit)
    return o.view(mixed.shape[0], layer.hv, layer.dv)


def gdn_commit(layer, mixed, a, b, qlens, slots, has_state, state, num_accepted_rows):
    meta = _Meta(qlens, slots, has_state, mixed.device, None, limit=list(num_accepted_rows))
    _run(layer, mixed, a, b, meta, state, True)


# ----------------------------------------------------------------------------- Mamba-2 (csrc/mamba2.cu)
_m2_bound = False


def _m2lib():
    global _m2_bound
    lib = _lib()
    if not _m2_bound:
        _f = C.c_float
        lib.atlas_conv1d_bias_silu.argtypes = [_vp, _ll, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _vp]
        lib.atlas_mamba2_scan.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _f, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _i,
                                          _i, _i, _i, _i, _i, _i, _vp]
        lib.atlas_mamba2_gated_norm.argtypes = [_vp, _ll, _vp, _ll, _vp, _vp, _ll, _i, _i, _i, _f, _vp]
        lib.atlas_relu2.argtypes = [_vp, _ll, _vp, _ll, _i, _i, _vp]
        _m2_bound = True
    return lib


def _mamba2_run(layer, xbc, dt, meta: _Meta, state, commit: bool):
    lib, st = _m2lib(), K._stream()
    K._dev(xbc)
    T, Cc = xbc.shape
    conv, h = state["conv"], state["h"]
    assert conv.dtype == torch.bfloat16 and h.dtype == torch.float32 and conv.is_contiguous() and h.is_contiguous()
    assert xbc.dtype == torch.bfloat16 and xbc.stride(1) == 1 and dt.stride(1) == 1
    y = torch.empty(T, Cc, dtype=torch.bfloat16, device=xbc.device)
    out = torch.empty(T, layer.d_inner, dtype=torch.bfloat16, device=xbc.device)
    cw = layer.conv_w if layer.conv_w.dtype == torch.bfloat16 else layer.conv_w.bfloat16()
    cb = None if layer.conv_b is None else (layer.conv_b if layer.conv_b.dtype == torch.bfloat16 else layer.conv_b.bfloat16())
    K._check(lib.atlas_conv1d_bias_silu(xbc.data_ptr(), xbc.stride(0), cw.data_ptr(), K._ptr(cb), Cc, layer.W, conv.data_ptr(),
                                        meta.seq_of.data_ptr(), meta.qsl.data_ptr(), meta.slots.data_ptr(), meta.has.data_ptr(),
                                        y.data_ptr(), Cc, T, st), "mamba2_conv")
    K._check(lib.atlas_mamba2_scan(y.data_ptr(), Cc, dt.data_ptr(), dt.stride(0), layer.A_log.data_ptr(), layer.D.data_ptr(),
                                   layer.dt_bias.data_ptr(), float(layer.cfg.mamba_dt_min), h.data_ptr(), out.data_ptr(),
                                   layer.d_inner, meta.qsl.data_ptr(), meta.slots.data_ptr(), meta.has.data_ptr(),
                                   K._ptr(meta.limit), meta.snap_rows.data_ptr(), meta.snap_slots.data_ptr(), meta.snaps, meta.B,
                                   layer.h, layer.p, layer.n, layer.g, 1 if commit else 0, st), "mamba2_scan")
    if commit:
        K._check(lib.atlas_gdn_conv_state(xbc.data_ptr(), xbc.stride(0), Cc, layer.W, conv.data_ptr(), meta.qsl.data_ptr(),
                                          meta.slots.data_ptr(), meta.has.data_ptr(), K._ptr(meta.limit),
                                          meta.snap_rows.data_ptr(), meta.snap_slots.data_ptr(), meta.snaps, meta.B, st),
                 "mamba2_conv_state")
    return out


def mamba2_forward(layer, xbc, dt, batch, state, commit):
    meta = getattr(batch, "_gdn_meta", None)
    if meta is None:
        meta = _Meta(batch.query_lens_host, batch.state_slots_host, batch.has_state_host, xbc.device, batch.snapshot_plan)
        batch._gdn_meta = meta
    return _mamba2_run(layer, xbc, dt, meta, state, commit)


def mamba2_commit(layer, xbc, dt, qlens, slots, has_state, state, num_accepted_rows):
    meta = _Meta(qlens, slots, has_state, xbc.device, None, limit=list(num_accepted_rows))
    _mamba2_run(layer, xbc, dt, meta, state, True)


def mamba2_gated_norm(y, z, w, group: int, eps: float):
    T, dI = y.shape
    out = torch.empty(T, dI, dtype=torch.bfloat16, device=y.device)
    wb = w if w.dtype == torch.bfloat16 else w.bfloat16()
    K._check(_m2lib().atlas_mamba2_gated_norm(y.data_ptr(), y.stride(0), z.data_ptr(), z.stride(0), wb.data_ptr(), out.data_ptr(),
                                              dI, T, dI // group, group, float(eps), K._stream()), "mamba2_gated_norm")
    return out


def relu_squared(x):
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    out = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
    K._dev(x2)
    K._check(_m2lib().atlas_relu2(x2.data_ptr(), x2.stride(0), out.data_ptr(), out.stride(0), x2.shape[0], x2.shape[1],
                                  K._stream()), "relu2")
    return out.view(x.shape)
