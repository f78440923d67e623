"""Bindings of the MoE, Gated-DeltaNet and NVFP4 parts of the kernel library."""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import cuda as K

_vp, _ll, _i, _f = C.c_void_p, C.c_longlong, C.c_int, C.c_float
FP8 = torch.float8_e4m3fn


def bind(lib) -> None:
    lib.atlas_moe_route.argtypes = [_vp, _ll, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp]
    lib.atlas_moe_align.argtypes = [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp]
    lib.atlas_moe_gather.argtypes = [_vp, _ll, _vp, _vp, _i, _i, _vp, _vp, _vp, _ll, _vp]
    lib.atlas_moe_combine.argtypes = [_vp, _ll, _vp, _vp, _i, _i, _i, _vp, _ll, _vp, _ll, _vp]
    lib.atlas_gemm_grouped.argtypes = [_i, _vp, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _i, _vp, _vp, _i, _vp, _vp]
    lib.atlas_moe_dispatch_prep.argtypes = [_vp, _i, _i, _i, _vp, _vp, _vp]
    lib.atlas_moe_dispatch_pack.argtypes = [_vp, _ll, _vp, _vp, _i, _i, _i, _vp, _i, _vp]
    lib.atlas_moe_recv_ids.argtypes = [_vp, _i, _i, _vp, _i, _i, _vp, _vp]
    lib.atlas_gemm_w4a16.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _i, _vp, _vp]
    lib.atlas_gemm_w4a16_grouped.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _i, _vp, _vp, _i, _vp, _vp]
    for name, args in _GDN_SIGS.items():
        if hasattr(lib, name):
            getattr(lib, name).argtypes = args


_GDN_SIGS = {}


# ----------------------------------------------------------------------------- NVFP4
def _row_gscale(gscale: torch.Tensor, rows: int) -> torch.Tensor:
    """The kernel takes one fp32 global scale per weight row; a checkpoint's scalar (or per-expert) scale is expanded
    once and cached.  The cache entry keeps the source tensor alive, so its address cannot be handed to another tensor
    while the entry exists."""
    key = (gscale.data_ptr(), rows)
    hit = _gs_cache.get(key)
    if hit is not None and hit[0] is gscale:
        return hit[1]
    g = gscale.float().reshape(-1)
    if g.numel() == 1:
        g = g.expand(rows)
    elif g.numel() != rows:
        g = g.repeat_interleave(rows // g.numel())
    g = g.contiguous()
    if len(_gs_cache) > 8192:
        _gs_cache.clear()
    _gs_cache[key] = (gscale, g)
    return g


_gs_cache = {}


def gemm_nvfp4(x, packed, bscale, gscale, out=None):
    """``x [M,K]`` bf16 times NVFP4 weights (packed ``[N,K/2]``, e4m3 ``[N,K/16]``, global scale): the weights stay
    packed in HBM and are widened to bf16 inside the kernel, tile by tile, on their way to the tensor cores."""
    M, Kd = x.shape
    N = packed.shape[0]
    if Kd % 64 != 0:                    # not a whole number of 64-wide slices: widen once and use the bf16 GEMM
        from .. import quant as Q
        hit = _nvfp4_cache.get(packed.data_ptr())
        if hit is None or hit[0] is not packed:
            hit = _nvfp4_cache[packed.data_ptr()] = (packed, Q.dequantize_nvfp4(packed, bscale, gscale).to(torch.bfloat16).contiguous())
        w = hit[1]
        return K.gemm_bf16(x if x.dtype == torch.bfloat16 else x.bfloat16(), w, out)
    d = K._dev(x)
    if x.dtype != torch.bfloat16:
        x = x.bfloat16()
    if x.stride(1) != 1:
        x = x.contiguous()
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    bs = bscale.view(torch.uint8)
    gs = _row_gscale(gscale, N)
    sms = K._num_sms[d]
    tiles_m = (M + 127) // 128
    bn = 128 if (N % 128 == 0 and tiles_m * (N // 128) >= sms) else 64
    K._check(K.lib().atlas_gemm_w4a16(x.data_ptr(), packed.data_ptr(), bs.data_ptr(), gs.data_ptr(), out.data_ptr(), M, N, Kd,
                                      x.stride(0), out.stride(0), bn, sms, K._status_ptr[d], K._stream()), "gemm_w4a16")
    return out


_nvfp4_cache = {}


# ----------------------------------------------------------------------------- MoE
_SCORE_MODES = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}


def moe_route(logits, top_k, norm_topk, scoring, bias=None, n_group=0, topk_group=0, scale=1.0, hash_table=None, token_ids=None):
    T, E = logits.shape
    K._dev(logits)
    if logits.dtype not in (torch.bfloat16, torch.float32):
        logits = logits.float()
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    plain = bias is None and hash_table is None and scale == 1.0 and not (n_group > 1 and 0 < topk_group < n_group)
    if plain and scoring in ("softmax", "sigmoid"):
        K._check(K.lib().atlas_moe_route(logits.data_ptr(), logits.stride(0), 1 if logits.dtype == torch.bfloat16 else 0, T, E,
                                         top_k, 1 if norm_topk else 0, 1 if scoring == "sigmoid" else 0, w.data_ptr(),
                                         ids.data_ptr(), K._stream()), "moe_route")
        return w, ids
    L = K.lib()
    if not getattr(L, "_route_ex_bound", False):
        L.atlas_moe_route_ex.argtypes = [_vp, _ll, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, C.c_float, _vp, _vp, _vp]
        L._route_ex_bound = True
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == E
    if hash_table is not None:
        assert hash_table.dtype == torch.int32 and hash_table.is_contiguous() and hash_table.shape[1] == top_k
        assert token_ids is not None and token_ids.dtype == torch.int32 and token_ids.numel() == T
    K._check(L.atlas_moe_route_ex(logits.data_ptr(), logits.stride(0), 1 if logits.dtype == torch.bfloat16 else 0, T, E, top_k,
                                  1 if norm_topk else 0, _SCORE_MODES[scoring], K._ptr(bias), int(n_group), int(topk_group),
                                  K._ptr(hash_table), K._ptr(token_ids), float(scale), w.data_ptr(), ids.data_ptr(), K._stream()),
             "moe_route_ex")
    return w, ids


def _expert_stacks(experts):
    """(kind, w13 [E*2I,H], s13, w2 [E*H,I], s2) in a layout the grouped GEMM takes."""
    cached = getattr(experts, "_gpu_stacks", None)
    if cached is not None:
        return cached
    if experts.kind == "fp8_block":
        out = (1, experts.w13.contiguous(), experts.w13_scale.contiguous().float(), experts.w2.contiguous(),
               experts.w2_scale.contiguous().float())
    elif experts.kind == "nvfp4" and experts.w13.shape[2] % 32 == 0 and experts.w2.shape[2] % 32 == 0:
        E, n1, n2 = experts.num_local, experts.w13.shape[1], experts.w2.shape[1]
        out = (2, experts.w13.contiguous(), (experts.w13_scale.contiguous().view(torch.uint8), _row_gscale(experts.w13_gscale, E * n1)),
               experts.w2.contiguous(), (experts.w2_scale.contiguous().view(torch.uint8), _row_gscale(experts.w2_gscale, E * n2)))
    else:
        w13, w2 = experts.dequantized() if experts.kind != "dense" else (experts.w13, experts.w2)
        out = (0, w13.to(torch.bfloat16).contiguous(), None, w2.to(torch.bfloat16).contiguous(), None)
        if experts.kind != "dense":
            experts._deq = None        # the bf16 stacks replace the fp32 dequantised copy
    experts._gpu_stacks = out
    return out


def moe_forward(x, topk_w, topk_ids, experts, e_lo, pctx, ep_mode, addend: Optional[torch.Tensor] = None):
    """Expert-sorted grouped FFN over this rank's experts.  Pairs routed to other ranks' experts contribute nothing
    here; with expert parallelism the partial outputs are summed across ranks (``allreduce`` mode, the default while
    activations are replicated across the group) or the rows travel to their experts and back (``alltoall`` mode)."""
    if ep_mode == "alltoall" and pctx is not None and pctx.ep_size > 1:
        comm = pctx.ep_comm if pctx.ep_comm is not None else pctx.comm
        if hasattr(comm, "all_to_all_rows"):
            out = _moe_forward_alltoall(x, topk_w, topk_ids, experts, e_lo, pctx, comm, addend)
            if out is not None:
                return out
    comm = None
    if pctx is not None and pctx.ep_size > 1:
        comm = pctx.ep_comm if pctx.ep_comm is not None else pctx.comm
    if comm is None:
        return _moe_local(x, topk_w, topk_ids, experts, e_lo, addend)
    # every rank runs its own experts on the replicated rows; the partial outputs are summed over the group.  With a
    # peer-memory backend and a decode-size step the weighted combine and that sum are ONE kernel.
    fused = comm if hasattr(comm, "moe_combine_all_reduce") else None
    out, reduced = _moe_local(x, topk_w, topk_ids, experts, e_lo, addend, fused_comm=fused, grouped=True)
    if not reduced:
        out = comm.all_reduce(out)
        if addend is not None:
            out = out + addend
    return out


def _moe_forward_alltoall(x, topk_w, topk_ids, experts, e_lo, pctx, comm, addend):
    """Dispatch / combine over peer memory.  Activations are replicated across the group, so rank r dispatches only its
    slice of the tokens: every (token, expert) pair is computed exactly once, on the rank that owns the expert.

    1. destination rank of every pair, segment offsets and positions (one kernel), rows packed with their expert id;
    2. all-to-all #1 (peer stores, device-side counts): rows arrive grouped by source rank;
    3. grouped expert FFN over the received rows (each row is one pair, weight 1);
    4. all-to-all #2 with the received offsets as send offsets: results return in the order they were sent;
    5. weighted sum over k (router probabilities) + addend at the source, then the token slices are put together.
    Returns None when the rows do not fit the symmetric slot (the caller falls back to the all-reduce form)."""
    T, H = x.shape
    k = topk_ids.shape[1]
    W, r = pctx.ep_size, pctx.ep_rank
    d = K._dev(x)
    dev = x.device
    lib, st = K.lib(), K._stream()
    per = (T + W - 1) // W
    t0, t1 = min(T, r * per), min(T, (r + 1) * per)
    Ts = t1 - t0
    pairs_cap = per * k                              # same on every rank: region capacity per source
    row_bytes = H * 2 + 16
    if (16 + pairs_cap * row_bytes) * W > comm.slot_bytes or H % 8:
        return None
    e_per_rank = experts.num_local
    ids = topk_ids[t0:t1].contiguous()
    w = topk_w[t0:t1].contiguous()
    send_off = torch.empty(W + 1, dtype=torch.int32, device=dev)
    pos = torch.empty(max(1, Ts * k), dtype=torch.int32, device=dev)
    K._check(lib.atlas_moe_dispatch_prep(ids.data_ptr(), Ts * k, e_per_rank, W, send_off.data_ptr(), pos.data_ptr(), st),
             "moe_dispatch_prep")
    send = torch.empty(max(1, Ts * k), row_bytes // 2, dtype=torch.bfloat16, device=dev)
    xs = x[t0:t1]
    if Ts:
        K._check(lib.atlas_moe_dispatch_pack(xs.data_ptr(), x.stride(0), ids.data_ptr(), pos.data_ptr(), Ts, k, H,
                                             send.data_ptr(), row_bytes, st), "moe_dispatch_pack")
    recv, recv_off = comm.all_to_all_rows(send, send_off, pairs_cap)
    cap = pairs_cap * W
    rid = torch.empty(cap, 1, dtype=torch.int32, device=dev)
    K._check(lib.atlas_moe_recv_ids(recv.data_ptr(), row_bytes, H, recv_off.data_ptr(), W, cap, rid.data_ptr(), st),
             "moe_recv_ids")
    ones = _ones(cap, dev)
    y_rows = _moe_local(recv[:, :H], ones, rid, experts, e_lo, None)          # [cap, H]; dead rows are zero
    back, _ = comm.all_to_all_rows(y_rows, recv_off, pairs_cap)
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    if Ts:
        ad = addend[t0:t1] if addend is not None else None
        K._check(lib.atlas_moe_combine(back.data_ptr(), H, pos.data_ptr(), w.data_ptr(), Ts, k, H, K._ptr(ad),
                                       addend.stride(0) if addend is not None else 0, out[t0:t1].data_ptr(), H, st),
                 "moe_combine_ep")
    return comm.all_reduce(out)             # slices are disjoint: the sum just places them


_ones_cache = {}


def _ones(n: int, dev) -> torch.Tensor:
    t = _ones_cache.get((n, dev))
    if t is None:
        t = _ones_cache[(n, dev)] = torch.ones(n, 1, dtype=torch.float32, device=dev)
    return t


_SMALL_MOE = os.environ.get("ATLAS_MOE_SMALL", "1") not in ("0", "false")
SMALL_MOE_ROWS_PER_EXPERT = 16


def _small_moe_ok(pairs: int, E: int, H: int, I: int) -> bool:
    return (_SMALL_MOE and pairs <= SMALL_MOE_ROWS_PER_EXPERT * E and H % 256 == 0 and I % 256 == 0)


def _bind_small(lib) -> None:
    if not getattr(lib, "_small_moe_bound", False):
        vp, i32, ll = C.c_void_p, C.c_int, C.c_longlong
        lib.atlas_moe_small_w4.argtypes = [i32, vp, ll, vp, vp, vp, i32, vp, vp, vp, vp, ll, i32, i32, vp]
        lib._small_moe_bound = True


def _finish(lib, y, slot_of, topk_w, T, k, H, addend, fused_comm, grouped, dev, st):
    """Weighted combine of the expert outputs.  ``grouped`` (expert-parallel caller): returns ``(out, reduced)``; the
    combine is fused with the group reduction (addend included) when the peer-memory backend takes the step, otherwise
    the local partial comes back WITHOUT the addend, which must be added once after the reduction."""
    if grouped and fused_comm is not None:
        out = fused_comm.moe_combine_all_reduce(y, slot_of, topk_w, T, k, addend)
        if out is not None:
            return out, True
    local_addend = None if grouped else addend
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    K._check(lib.atlas_moe_combine(y.data_ptr(), H, slot_of.data_ptr(), topk_w.data_ptr(), T, k, H, K._ptr(local_addend),
                                   local_addend.stride(0) if local_addend is not None else 0, out.data_ptr(), H, st), "moe_combine")
    return (out, False) if grouped else out


def _moe_local(x, topk_w, topk_ids, experts, e_lo, addend: Optional[torch.Tensor] = None, fused_comm=None, grouped=False):
    if K.checked.ENABLED:
        K.checked.index_range("topk_ids", topk_ids, 0, 1 << 20)
        K.checked.finite("topk_w", topk_w)
    """Local experts only: align -> gather (+quant) -> grouped GEMM -> SiLU*mul -> grouped GEMM -> weighted combine."""
    T, H = x.shape
    k = topk_ids.shape[1]
    d = K._dev(x)
    dev = x.device
    kind, w13, s13, w2, s2 = _expert_stacks(experts)
    E = experts.num_local
    N1, I = w13.shape[1], (w2.shape[2] * 2 if kind == 2 else w2.shape[2])
    max_rows = ((T * k + E * 127 + 127) // 128) * 128
    max_rows = min(max_rows, ((T * k + 127) // 128 + E) * 128)
    lib, st, sms, status = K.lib(), K._stream(), K._num_sms[d], K._status_ptr[d]
    slot_of = torch.empty(T * k, dtype=torch.int32, device=dev)
    row_token = torch.empty(max_rows, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(max_rows // 128, dtype=torch.int32, device=dev)
    num_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    K._check(lib.atlas_moe_align(topk_ids.data_ptr(), T, k, e_lo, E, slot_of.data_ptr(), row_token.data_ptr(),
                                 tile_expert.data_ptr(), num_tiles.data_ptr(), max_rows, status, st), "moe_align")

    def bn_for(n):
        return 128 if n % 128 == 0 else 64

    if kind == 2 and _small_moe_ok(T * k, E, H, I):
        # decode-size batch on NVFP4 experts: a few rows per expert, so stream the weights through the register-level
        # dequant kernel (rows gathered by token inside it, SiLU fused) instead of 128-row tcgen05 tiles
        _bind_small(lib)
        act = torch.empty(max_rows, I, dtype=torch.bfloat16, device=dev)
        K._check(lib.atlas_moe_small_w4(1, x.data_ptr(), x.stride(0), row_token.data_ptr(), tile_expert.data_ptr(),
                                        num_tiles.data_ptr(), max_rows // 128, w13.data_ptr(), s13[0].data_ptr(),
                                        s13[1].data_ptr(), act.data_ptr(), I, H, 2 * I, st), "moe_small_gate_up")
        y = torch.empty(max_rows, H, dtype=torch.bfloat16, device=dev)
        K._check(lib.atlas_moe_small_w4(0, act.data_ptr(), I, row_token.data_ptr(), tile_expert.data_ptr(),
                                        num_tiles.data_ptr(), max_rows // 128, w2.data_ptr(), s2[0].data_ptr(),
                                        s2[1].data_ptr(), y.data_ptr(), H, I, H, st), "moe_small_down")
        return _finish(lib, y, slot_of, topk_w, T, k, H, addend, fused_comm, grouped, dev, st)
    if kind == 1:
        xq = torch.empty(max_rows, H, dtype=FP8, device=dev)
        xs = torch.empty(H // 128, max_rows, dtype=torch.float32, device=dev)
        K._check(lib.atlas_moe_gather(x.data_ptr(), x.stride(0), row_token.data_ptr(), num_tiles.data_ptr(), max_rows, H,
                                      None, xq.data_ptr(), xs.data_ptr(), max_rows, st), "moe_gather")
        a1, a1s = xq, xs
    else:
        xp = torch.empty(max_rows, H, dtype=torch.bfloat16, device=dev)
        K._check(lib.atlas_moe_gather(x.data_ptr(), x.stride(0), row_token.data_ptr(), num_tiles.data_ptr(), max_rows, H,
                                      xp.data_ptr(), None, None, 0, st), "moe_gather")
        a1, a1s = xp, None
    h1 = torch.empty(max_rows, 2 * I, dtype=torch.bfloat16, device=dev)
    if kind == 2:
        K._check(lib.atlas_gemm_w4a16_grouped(a1.data_ptr(), w13.data_ptr(), s13[0].data_ptr(), s13[1].data_ptr(), h1.data_ptr(),
                                              max_rows, 2 * I, H, E, H, 2 * I, bn_for(2 * I), tile_expert.data_ptr(),
                                              num_tiles.data_ptr(), sms, status, st), "moe_gemm1_w4")
    else:
        K._check(lib.atlas_gemm_grouped(kind, a1.data_ptr(), w13.data_ptr(), h1.data_ptr(), K._ptr(a1s), max_rows, K._ptr(s13),
                                        max_rows, 2 * I, H, E, H, H, 2 * I, bn_for(2 * I), tile_expert.data_ptr(),
                                        num_tiles.data_ptr(), sms, status, st), "moe_gemm1")
    if kind == 1:
        aq = torch.empty(max_rows, I, dtype=FP8, device=dev)
        asc = torch.empty(I // 128, max_rows, dtype=torch.float32, device=dev)
        K._check(lib.atlas_silu_mul(h1.data_ptr(), 2 * I, max_rows, I, None, 0, aq.data_ptr(), I, asc.data_ptr(), max_rows,
                                    num_tiles.data_ptr(), st), "moe_silu")
        a2, a2s = aq, asc
    else:
        act = torch.empty(max_rows, I, dtype=torch.bfloat16, device=dev)
        K._check(lib.atlas_silu_mul(h1.data_ptr(), 2 * I, max_rows, I, act.data_ptr(), I, None, 0, None, 0,
                                    num_tiles.data_ptr(), st), "moe_silu")
        a2, a2s = act, None
    y = torch.empty(max_rows, H, dtype=torch.bfloat16, device=dev)
    if kind == 2:
        K._check(lib.atlas_gemm_w4a16_grouped(a2.data_ptr(), w2.data_ptr(), s2[0].data_ptr(), s2[1].data_ptr(), y.data_ptr(),
                                              max_rows, H, I, E, I, H, bn_for(H), tile_expert.data_ptr(), num_tiles.data_ptr(),
                                              sms, status, st), "moe_gemm2_w4")
    else:
        K._check(lib.atlas_gemm_grouped(kind, a2.data_ptr(), w2.data_ptr(), y.data_ptr(), K._ptr(a2s), max_rows, K._ptr(s2),
                                        max_rows, H, I, E, I, I, H, bn_for(H), tile_expert.data_ptr(), num_tiles.data_ptr(),
                                        sms, status, st), "moe_gemm2")
    return _finish(lib, y, slot_of, topk_w, T, k, H, addend, fused_comm, grouped, dev, st)


# ----------------------------------------------------------------------------- GDN (bound when gdn.cu is present)
def gdn_forward(layer, mixed, a, b, batch, state, commit):
    from . import cuda_gdn
    return cuda_gdn.gdn_forward(layer, mixed, a, b, batch, state, commit)


def gdn_commit(layer, mixed, a, b, qlens, slots, has_state, state, num_accepted_rows):
    from . import cuda_gdn
    return cuda_gdn.gdn_commit(layer, mixed, a, b, qlens, slots, has_state, state, num_accepted_rows)
