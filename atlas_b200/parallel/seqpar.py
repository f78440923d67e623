"""Sequence-parallel tensor parallelism for prefill-size steps: GEMM -> reduce-scatter and all-gather -> GEMM over
NVLink peer memory, with the residual stream sharded by rows.

Per layer half (attention, FFN) the three kernels are

1. ``gemm_rs``       row-parallel GEMM (o_proj / down_proj) whose epilogue stores every bf16 partial tile straight into
                     the memory of the rank that owns the row block (``csrc/gemm.cu``, reduce-scatter epilogue);
2. ``reduce_norm``   on the owner: sum of the partials in rank order + residual shard + RMSNorm weight + FP8 group
                     quantisation, rows and scales stored into every rank's gathered buffer (``csrc/seqpar.cu``);
3. the next column-parallel GEMM (qkv / gate_up), whose TMA producer polls the per-row-group arrival flags of the
   gathered buffer before it loads a tile (``csrc/gemm.cu``, ``atlas_gemm_gathered``).

Dependencies only run forwards (1 -> 2 -> 3), so the ranks of a group can also be executed one after another on a
single GPU, which is how the numerics test covers the multi-rank path on one device.

One :class:`SeqParallelArea` holds a rank's buffers; ``connect`` receives every rank's base pointer.  With processes on
several GPUs the base pointers come from CUDA IPC (:meth:`SymmBackend.seq_parallel`).

Reference counterpart: the bf16 all-reduce after o_proj / down_proj
(``crates/spark-model/src/layers/qwen3_attention/trait_impl/prefill_inner.rs:194``) and the backend's unused
``all_gather`` / ``reduce_scatter`` verbs (``crates/spark-comm/src/nccl_backend/comm_impl.rs:139-175``).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch

_vp, _i, _ll, _sz, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t, C.c_float
ROWS_PER_FLAG = 8


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class _Raw:
    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": tuple(shape), "typestr": typestr, "version": 2,
                                         "strides": None}


def device_view(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    """A torch tensor aliasing raw device memory."""
    if dtype == torch.bfloat16:
        return torch.as_tensor(_Raw(ptr, shape, "<i2"), device=device).view(torch.bfloat16)
    if dtype == torch.float8_e4m3fn:
        return torch.as_tensor(_Raw(ptr, shape, "|u1"), device=device).view(torch.float8_e4m3fn)
    if dtype == torch.float32:
        return torch.as_tensor(_Raw(ptr, shape, "<f4"), device=device)
    if dtype == torch.int32:
        return torch.as_tensor(_Raw(ptr, shape, "<i4"), device=device)
    raise ValueError(dtype)


def partition(T: int, world: int) -> Tuple[int, int]:
    """(128-row blocks owned by each rank, rows per rank) for a step of ``T`` rows.  A step of at most 128 rows (decode)
    is owned row by row instead: every rank gets the same multiple of eight rows of the single block, so that all ranks
    share the reduce + norm work of a decode step (``fine_rows``)."""
    fine = fine_rows(T, world)
    if fine:
        return 1, fine
    tiles = (T + 127) // 128
    tpr = (tiles + world - 1) // world
    return tpr, tpr * 128


def fine_rows(T: int, world: int) -> int:
    """Rows per rank under row-level ownership, or 0 when the step is owned in 128-row blocks."""
    if T > 128 or world < 2:
        return 0
    return ((T + world - 1) // world + ROWS_PER_FLAG - 1) // ROWS_PER_FLAG * ROWS_PER_FLAG


class SeqParallelArea:
    """One rank's buffers of the sequence-parallel path, sized for ``max_tokens`` rows of width ``hidden``.

    Layout of the single allocation (identical offsets on every rank):
    ``[partials: world x rows_cap x H bf16][gathered fp8 rows: T_pad x H][gathered scales: H/128 x T_pad fp32]``
    ``[gathered bf16 rows: T_pad x H][reduce-scatter flags][arrival flags]``.
    """

    def __init__(self, rank: int, world: int, max_tokens: int, hidden: int, device, wait_cycles: int = 0):
        from ..ops import cuda as K
        self.K, self.lib = K, K.lib()
        self.rank, self.world, self.H, self.device = rank, world, hidden, torch.device(device)
        self.wait_cycles = int(wait_cycles)
        assert hidden % 256 == 0 and 1 <= world <= 8
        self.t_pad = _align(max(max_tokens, 128), 128)
        tpr = ((self.t_pad + 127) // 128 + world - 1) // world       # capacity by the 128-row block rule (covers row-level ownership)
        rows_cap = tpr * 128
        self.rows_cap = rows_cap
        self.part_stride = _align(rows_cap * hidden * 2)
        self.flag_words_rs = tpr * (hidden // 64) * 8
        self.flag_words_ag = self.t_pad // ROWS_PER_FLAG
        off = 0
        self.off_part = off; off += world * self.part_stride
        self.off_agq = off; off += _align(self.t_pad * hidden)
        self.off_ags = off; off += _align((hidden // 128) * self.t_pad * 4)
        self.off_agh = off; off += _align(self.t_pad * hidden * 2)
        self.off_rsf = off; off += _align(self.flag_words_rs * 4)
        self.off_agf = off; off += _align(self.flag_words_ag * 4)
        self.nbytes = off
        self.base = 0                       # set by the owner of the memory (allocate / adopt)
        self._keep = None
        self.rs_state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.ag_state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.row_counters = torch.zeros(rows_cap // ROWS_PER_FLAG + 1, dtype=torch.int32, device=self.device)
        self.peers: List[int] = []
        self._bind()
        self.calls = {"gemm_rs": 0, "reduce_norm": 0, "reduce_hidden": 0}

    def _bind(self) -> None:
        lib = self.lib
        if getattr(lib, "_sp_bound", False):
            return
        lib.atlas_gemm_reduce_scatter.argtypes = [_i, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _ll, _ll, _i, C.POINTER(_vp),
                                                  C.POINTER(_vp), _i, _i, _vp, _sz, _i, _sz, _i, _ll, _vp, _vp, C.POINTER(_i), _i]
        lib.atlas_sp_reduce_norm_gather.argtypes = [_i, _vp, _sz, _vp, _vp, _i, _vp, _vp, _i, _f, C.POINTER(_vp), C.POINTER(_vp),
                                                    _ll, C.POINTER(_vp), C.POINTER(_vp), _vp, _i, _i, _i, _i, _i, _ll, _vp, _vp, _vp]
        lib.atlas_sp_wait_rows.argtypes = [_vp, _vp, _i, _ll, _vp, _vp]
        lib._sp_bound = True

    # ------------------------------------------------------------------ memory
    def allocate_local(self) -> int:
        """Plain device memory (single-process use: tests that run the ranks of a group one after another)."""
        self._keep = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
        self.base = self._keep.data_ptr()
        return self.base

    def adopt(self, base_ptr: int) -> None:
        """Use memory obtained elsewhere (a symmetric allocation exported over CUDA IPC); must be zero-filled."""
        self.base = int(base_ptr)

    def connect(self, bases: List[int]) -> None:
        """``bases[r]`` = address, in this process, of rank r's area (own entry = ``self.base``)."""
        assert len(bases) == self.world and bases[self.rank] == self.base
        self.peers = [int(b) for b in bases]

        def arr(off):
            vals = [b + off for b in self.peers] + [None] * (8 - self.world)
            return (_vp * 8)(*vals)
        self.a_part, self.a_agq, self.a_ags = arr(self.off_part), arr(self.off_agq), arr(self.off_ags)
        self.a_agh, self.a_rsf, self.a_agf = arr(self.off_agh), arr(self.off_rsf), arr(self.off_agf)

    # ------------------------------------------------------------------ kernels
    def _row_range(self, T: int) -> Tuple[int, int, int]:
        tpr, rows = partition(T, self.world)
        row0 = self.rank * rows
        return tpr, row0, max(0, min(T - row0, rows))

    def residual_shard(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's rows of a replicated ``[T, H]`` tensor, as a private contiguous copy."""
        _, row0, n = self._row_range(x.shape[0])
        return x[row0:row0 + n].clone() if n else x[:0].clone()

    def gemm_rs(self, act, w) -> None:
        """Row-parallel GEMM on this rank's K-shard; partial tiles go to the row owners."""
        K = self.K
        if w.kind == "fp8_block":
            q, sc = act.fp8()
            kind, a, a_scale, b, b_scale = 1, q, sc, w.weight, w.scale
            if sc.stride(0) != 1 or sc.stride(1) % 4 or sc.stride(1) < (q.shape[0] + 127) // 128 * 128 or sc.data_ptr() % 16:
                a_scale = K._scale_buf(q.shape[0], sc.shape[1], q.device)
                a_scale.copy_(sc)
        elif w.kind == "dense" and w.weight.dtype == torch.bfloat16:
            kind, a, a_scale, b, b_scale = 0, act.plain(), None, w.weight, None
        else:
            raise ValueError(f"sequence-parallel GEMM: unsupported weight kind {w.kind}")
        T, Kd = a.shape
        N = b.shape[0]
        assert N == self.H and T <= self.t_pad and a.stride(1) == 1
        d = K._dev(a)
        sms = K._num_sms[d]
        tpr, _, _ = self._row_range(T)
        m_tiles = (T + 127) // 128
        if kind == 1 and N % 256 == 0 and m_tiles * (N // 256) >= sms:
            bn = 256                # prefill-size FP8: the wide tile (see ops.cuda.gemm_plan)
        else:
            bn = 128 if m_tiles * (N // 128) >= sms else 64
        nt = _i(0)
        rc = self.lib.atlas_gemm_reduce_scatter(kind, a.data_ptr(), b.data_ptr(), K._ptr(a_scale),
                                                a_scale.stride(1) if a_scale is not None else 0, K._ptr(b_scale),
                                                b_scale.shape[1] if b_scale is not None else 0, T, N, Kd, a.stride(0),
                                                b.stride(0), bn, self.a_part, self.a_rsf, self.rank, self.world,
                                                self.rs_state.data_ptr(), self.part_stride, tpr, self.flag_words_rs, sms,
                                                self.wait_cycles, K._status_ptr[d], K._stream(), C.byref(nt),
                                                fine_rows(T, self.world))
        K._check(rc, "gemm_reduce_scatter")
        self._n_tiles, self._T = nt.value, T
        self.calls["gemm_rs"] += 1

    def _reduce(self, mode: int, residual: Optional[torch.Tensor], norm_w, eps: float, plus_one: bool) -> None:
        K = self.K
        T = self._T
        _, row0, rows_own = self._row_range(T)
        d = K._dev(self.rs_state)
        if residual is not None:
            assert residual.is_contiguous() and residual.dtype == torch.bfloat16 and residual.shape == (rows_own, self.H)
        rc = self.lib.atlas_sp_reduce_norm_gather(mode, self.base + self.off_part, self.part_stride, self.base + self.off_rsf,
                                                  self.rs_state.data_ptr(), self._n_tiles,
                                                  residual.data_ptr() if (residual is not None and rows_own) else None,
                                                  K._ptr(norm_w), 1 if plus_one else 0, float(eps), self.a_agq, self.a_ags,
                                                  self.t_pad, self.a_agh, self.a_agf, self.ag_state.data_ptr(), self.rank,
                                                  self.world, self.H, row0, rows_own, self.wait_cycles, K._status_ptr[d],
                                                  K._stream(), self.row_counters.data_ptr() if fine_rows(T, self.world) else None)
        K._check(rc, "sp_reduce_norm_gather")

    def reduce_norm(self, residual: torch.Tensor, norm_w: torch.Tensor, eps: float, plus_one: bool = False):
        """Owner-side reduce + residual + RMSNorm + FP8 quantisation, gathered to every rank.  Returns the gathered
        activations as an :class:`~atlas_b200.ops.Act` whose rows may still be in flight: the consuming GEMM waits on
        the arrival flags (``Act.ready``)."""
        from ..ops import Act
        assert norm_w.dtype == torch.bfloat16 and norm_w.is_contiguous()
        self._reduce(0, residual, norm_w, eps, plus_one)
        self.calls["reduce_norm"] += 1
        T = self._T
        q = device_view(self.base + self.off_agq, (self.t_pad, self.H), torch.float8_e4m3fn, self.device)[:T]
        s = device_view(self.base + self.off_ags, (self.H // 128, self.t_pad), torch.float32, self.device)[:, :T].t()
        return Act(q=q, s=s, dtype=torch.bfloat16,
                   ready=(self.base + self.off_agf, self.ag_state.data_ptr(), self.wait_cycles))

    def reduce_hidden(self, residual: torch.Tensor) -> torch.Tensor:
        """Owner-side reduce + residual, bf16 rows gathered to every rank; returns the complete ``[T, H]`` tensor."""
        self.reduce_hidden_start(residual)
        return self.hidden_wait()

    def reduce_hidden_start(self, residual: torch.Tensor) -> None:
        """First half of :meth:`reduce_hidden`: this rank's rows go out, nothing is waited for."""
        self._reduce(1, residual, None, 0.0, False)

    def hidden_wait(self) -> torch.Tensor:
        """Second half: a kernel that returns once every rank's rows of the last hidden gather have arrived."""
        K = self.K
        T = self._T
        d = K._dev(self.rs_state)
        K._check(self.lib.atlas_sp_wait_rows(self.base + self.off_agf, self.ag_state.data_ptr(), T, self.wait_cycles,
                                             K._status_ptr[d], K._stream()), "sp_wait_rows")
        self.calls["reduce_hidden"] += 1
        return device_view(self.base + self.off_agh, (self.t_pad, self.H), torch.bfloat16, self.device)[:T]
