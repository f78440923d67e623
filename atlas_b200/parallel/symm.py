"""SymmBackend: collectives executed by this engine's own kernels over NVLink peer memory.

Every rank allocates one symmetric region (two data slots, a flag area, a small state block), exports it with CUDA
IPC and maps all peers' regions; the kernels of ``csrc/comm.cu`` then move data with plain peer loads / stores and
synchronise with release/acquire flags (bounded waits).  Anything the kernels do not cover (odd sizes, dtypes other
than bf16, messages larger than a slot) goes to the wrapped ``torch.distributed`` backend, which is also used for the
bootstrap exchange of IPC handles.

A rank that stops participating makes the others' waits expire: the kernel returns, the device status word is set,
and :meth:`check` poisons the communicator (same contract as ``poison_on_error`` in
``crates/spark-comm/src/collective_wait.rs``).
"""
from __future__ import annotations

import os

import ctypes as C
from typing import List, Optional

import torch

from .comm import CommBackend, CommError, TorchDistBackend

_vp, _i, _ll, _sz = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t
ONESHOT_MAX_BYTES = 2 << 20
P2P_MAX_BYTES = int(os.environ.get("ATLAS_P2P_MAX_BYTES", str(64 << 20)))   # larger messages go to the bootstrap backend
FUSED_DECODE_MAX_K = 4096
FUSED_MAX_OUT_BYTES = 2 << 20    # the fused GEMM+all-reduce pays off for decode-size outputs
# one-shot form of the fused kernel (partials pushed to every peer) while the pushed bytes per rank stay below this
FUSED_ONESHOT_MAX_PUSH_BYTES = int(os.environ.get("ATLAS_FUSED_ONESHOT_MAX", str(8 << 20)))


class SymmBackend(CommBackend):
    name = "symm-p2p"

    def __init__(self, base: TorchDistBackend, device: torch.device, slot_bytes: int = 160 << 20, blocks: int = 64,
                 wait_cycles: int = 0, fused_bytes: int = 192 << 20):
        from ..ops import cuda as K
        self.K = K
        self.base, self.device = base, device
        self.rank, self.world_size = base.rank, base.world_size
        self.slot_bytes, self.blocks, self.wait_cycles = int(slot_bytes), int(blocks), int(wait_cycles)
        self.lib = K.lib()
        lib = self.lib
        lib.atlas_symm_alloc.argtypes = [_sz, C.POINTER(_vp)]
        lib.atlas_ipc_export.argtypes = [_vp, C.c_char_p]
        lib.atlas_ipc_open.argtypes = [C.c_char_p, C.POINTER(_vp)]
        lib.atlas_ipc_close.argtypes = [_vp]
        lib.atlas_symm_free.argtypes = [_vp]
        lib.atlas_allreduce_bf16.argtypes = [_i, C.POINTER(_vp), C.POINTER(_vp), _i, _i, _vp, _vp, _sz, _sz, _vp, _i, _vp, _ll, _vp]
        lib.atlas_alltoall_rows.argtypes = [C.POINTER(_vp), C.POINTER(_vp), _i, _i, _vp, _vp, _vp, _vp, _i, _i, _sz, _vp, _i, _vp,
                                            _ll, _vp]
        torch.cuda.set_device(device)
        self.dev_index = K._dev(torch.empty(1, device=device))
        self.sms = K._num_sms[self.dev_index]
        flag_bytes = 2 * 256 * 8 * 4
        self._data = self._alloc(2 * self.slot_bytes)
        self._flags = self._alloc(flag_bytes)
        self.state = torch.zeros(4, dtype=torch.int32, device=device)
        handles = [None] * self.world_size
        mine = (self._export(self._data), self._export(self._flags))
        base.dist.all_gather_object(handles, mine, group=base.group)
        self._opened: List[int] = []
        data_ptrs, flag_ptrs = [], []
        for r, (hd, hf) in enumerate(handles):
            if r == self.rank:
                data_ptrs.append(self._data)
                flag_ptrs.append(self._flags)
            else:
                data_ptrs.append(self._open(hd))
                flag_ptrs.append(self._open(hf))
        self.data_arr = (_vp * 8)(*(data_ptrs + [None] * (8 - len(data_ptrs))))
        self.flag_arr = (_vp * 8)(*(flag_ptrs + [None] * (8 - len(flag_ptrs))))
        # dedicated area of the fused GEMM+all-reduce (partials from every rank + the result), its flags and epoch state
        self.fused_bytes = int(fused_bytes)
        self.max_tiles = 16384
        self._fdata = self._alloc(self.fused_bytes)
        self._fflags = self._alloc((self.max_tiles * 17) * 4)
        self.fstate = torch.zeros(4, dtype=torch.int32, device=device)
        fh = [None] * self.world_size
        base.dist.all_gather_object(fh, (self._export(self._fdata), self._export(self._fflags)), group=base.group)
        fd, ff = [], []
        for r, (hd, hf) in enumerate(fh):
            fd.append(self._fdata if r == self.rank else self._open(hd))
            ff.append(self._fflags if r == self.rank else self._open(hf))
        self.fdata_arr = (_vp * 8)(*(fd + [None] * (8 - len(fd))))
        self.fflag_arr = (_vp * 8)(*(ff + [None] * (8 - len(ff))))
        lib.atlas_gemm_allreduce.argtypes = [_i, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _ll, _ll, _i, C.POINTER(_vp),
                                             C.POINTER(_vp), _i, _i, _vp, _sz, _i, C.POINTER(_sz), _i, _ll, _vp, _vp,
                                             _i, _vp, _ll, _i, _vp, _vp, _vp]
        base.barrier()
        self._sp_areas, self._sp_mem = {}, []
        self.sp_min_capacity = int(os.environ.get("ATLAS_SP_MIN_CAPACITY", "8192"))
        self.calls = {"oneshot": 0, "twoshot": 0, "alltoall": 0, "fallback": 0, "gemm_allreduce": 0, "gemm_allreduce_oneshot": 0}

    # ------------------------------------------------------------------ IPC plumbing
    def _alloc(self, nbytes: int) -> int:
        p = _vp()
        if self.lib.atlas_symm_alloc(nbytes, C.byref(p)) != 0:
            raise CommError(f"symmetric allocation of {nbytes} bytes failed")
        return p.value

    def _export(self, ptr: int) -> bytes:
        buf = C.create_string_buffer(64)
        if self.lib.atlas_ipc_export(ptr, buf) <= 0:
            raise CommError("cudaIpcGetMemHandle failed")
        return buf.raw

    def _open(self, handle: bytes) -> int:
        p = _vp()
        if self.lib.atlas_ipc_open(handle, C.byref(p)) != 0:
            raise CommError("cudaIpcOpenMemHandle failed (are the GPUs peer-accessible?)")
        self._opened.append(p.value)
        return p.value

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self.lib.atlas_ipc_close(p)
        self._opened = []
        for p in [self._data, self._flags, self._fdata, self._fflags] + self._sp_mem:
            if p:
                self.lib.atlas_symm_free(p)
        self._sp_mem, self._sp_areas = [], {}
        self._data = self._flags = 0

    def check(self) -> None:
        """Synchronise, read the device status word, poison on an expired wait."""
        st = self.K.check_status(self.dev_index)
        if st:
            self.poison(f"peer wait expired (status {st:#x})")
            raise CommError(f"collective wait expired on rank {self.rank} (status {st:#x})")

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        self._guard()
        nbytes = t.numel() * t.element_size()
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or nbytes % 16 or nbytes == 0:
            self.calls["fallback"] += 1
            return self.base.all_reduce(t)
        if nbytes <= min(ONESHOT_MAX_BYTES, self.slot_bytes):
            kind = 0
        elif 2 * nbytes <= self.slot_bytes and nbytes <= P2P_MAX_BYTES:
            kind = 1
        else:
            self.calls["fallback"] += 1
            return self.base.all_reduce(t)
        self.calls["oneshot" if kind == 0 else "twoshot"] += 1
        K = self.K
        # every block pays one flag exchange per peer; the two-shot form wants every SM streaming
        blocks = max(1, min(self.blocks, nbytes // 16384)) if kind == 0 else max(1, min(self.sms, 256, nbytes // 65536))
        rc = self.lib.atlas_allreduce_bf16(kind, self.data_arr, self.flag_arr, self.rank, self.world_size, t.data_ptr(),
                                           t.data_ptr(), nbytes, self.slot_bytes, self.state.data_ptr(), blocks,
                                           K._status_ptr[self.dev_index], self.wait_cycles, K._stream())
        K._check(rc, "allreduce_p2p")
        return t

    def all_to_all_rows(self, rows: torch.Tensor, send_off: torch.Tensor, max_recv_rows: int):
        """``rows [R, W]`` (any 16-byte-multiple row size), ``send_off [world+1]`` int32 on the device.  Returns
        ``(recv_rows [max_recv_rows, W], recv_off [world+1])``; no host synchronisation."""
        self._guard()
        K = self.K
        row_bytes = rows.shape[1] * rows.element_size()
        region_rows = max_recv_rows
        assert rows.is_contiguous() and row_bytes % 16 == 0
        assert (16 + region_rows * row_bytes) * self.world_size <= self.slot_bytes, "all-to-all exceeds the symmetric slot"
        out = torch.empty(max_recv_rows * self.world_size, rows.shape[1], dtype=rows.dtype, device=rows.device)
        recv_off = torch.empty(self.world_size + 1, dtype=torch.int32, device=rows.device)
        self.calls["alltoall"] += 1
        rc = self.lib.atlas_alltoall_rows(self.data_arr, self.flag_arr, self.rank, self.world_size, rows.data_ptr(),
                                          send_off.data_ptr(), out.data_ptr(), recv_off.data_ptr(), row_bytes, region_rows,
                                          self.slot_bytes, self.state.data_ptr(), min(self.blocks, self.sms), K._status_ptr[self.dev_index],
                                          self.wait_cycles, K._stream())
        K._check(rc, "alltoall_rows")
        return out, recv_off

    def moe_combine_all_reduce(self, y: torch.Tensor, slot_of: torch.Tensor, topk_w: torch.Tensor, T: int, k: int,
                               addend: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Weighted top-k combine of this rank's expert outputs fused with the sum over the group (one kernel).
        Returns None when the step is too large for the one-exchange form (the caller combines, then all-reduces)."""
        self._guard()
        H = y.shape[1]
        nbytes = T * H * 2
        if y.dtype != torch.bfloat16 or H % 8 or nbytes > min(ONESHOT_MAX_BYTES, self.slot_bytes) or y.stride(1) != 1:
            return None
        K = self.K
        if not getattr(self.lib, "_mca_bound", False):
            self.lib.atlas_moe_combine_allreduce.argtypes = [C.POINTER(_vp), C.POINTER(_vp), _i, _i, _vp, _ll, _vp, _vp, _i, _i, _i,
                                                             _vp, _ll, _vp, _ll, _sz, _vp, _i, _vp, _ll, _vp]
            self.lib._mca_bound = True
        out = torch.empty(T, H, dtype=torch.bfloat16, device=y.device)
        blocks = max(1, min(self.blocks, nbytes // 16384))
        rc = self.lib.atlas_moe_combine_allreduce(self.data_arr, self.flag_arr, self.rank, self.world_size, y.data_ptr(),
                                                  y.stride(0), slot_of.data_ptr(), topk_w.data_ptr(), T, k, H, K._ptr(addend),
                                                  addend.stride(0) if addend is not None else 0, out.data_ptr(), H,
                                                  self.slot_bytes, self.state.data_ptr(), blocks,
                                                  K._status_ptr[self.dev_index], self.wait_cycles, K._stream())
        K._check(rc, "moe_combine_allreduce")
        self.calls["moe_combine_allreduce"] = self.calls.get("moe_combine_allreduce", 0) + 1
        return out

    def gemm_allreduce(self, act, w, epilogue=None):
        """``sum over ranks of (act_shard @ W_shard^T)`` with the reduction fused into the GEMM kernel.  Returns a
        view of the result inside this rank's fused area (valid until the next fused call), or None when the
        shape is not covered and the caller should use GEMM + all_reduce.

        ``epilogue = (residual, norm_w, plus_one)`` (one-shot form, FP8 weights only): the kernel also adds the sum to
        ``residual`` in place and returns ``(q, scales, (row sums of squares, parts))``, the FP8 form of
        ``residual * norm_w`` with the row's 1/rms factor left to the consumer, instead of the bf16 sum; None when the
        shape is not covered (nothing has been launched then)."""
        self._guard()
        K = self.K
        if epilogue is not None and (w.kind != "fp8_block" or w.weight.shape[0] % 128):
            return None
        if w.kind == "fp8_block":
            q, sc = act.fp8()
            kind, a, a_scale, b, b_scale = 1, q, sc, w.weight, w.scale
            if sc.stride(0) != 1 or sc.stride(1) % 4 or sc.stride(1) < (q.shape[0] + 127) // 128 * 128:
                fixed = K._scale_buf(q.shape[0], sc.shape[1], q.device)
                fixed.copy_(sc)
                a_scale = fixed
        elif w.kind == "dense" and w.weight.dtype == torch.bfloat16:
            kind, a, a_scale, b, b_scale = 0, act.plain(), None, w.weight, None
        else:
            return None
        M, Kd = a.shape
        N = b.shape[0]
        if N % 8 or a.stride(1) != 1 or M * N * 2 > FUSED_MAX_OUT_BYTES:
            return None
        sms = K._num_sms[self.dev_index]
        oneshot = M * N * 2 * (self.world_size - 1) <= FUSED_ONESHOT_MAX_PUSH_BYTES
        ws = cnt = out = None
        splits = 1
        if oneshot:
            # every rank pushes its partial tiles to all peers and sums locally: one flag exchange, K may be split
            if epilogue is not None:
                bn, splits = K.fused_block_n(2, M, N, Kd, sms)
                bn = 128
            else:
                bn, splits = K.gemm_plan(M, N, Kd, kind, sms)
                bn = min(bn, 128)
            tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
            need = 4 * self.world_size * tiles * 128 * bn * 2 + 1024
            if splits > 1:
                ws = K.scratch("gemm_ws", K._GEMM_WS_BYTES, a.device)
                cnt = K.scratch("gemm_counters", 1 << 18, a.device)
            if epilogue is None:
                out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
        else:
            if epilogue is not None:
                return None
            if M <= 128 and Kd > FUSED_DECODE_MAX_K:
                # decode-size rows with a long K and an output too large for the one-shot form: the two-shot kernel has
                # no split-K, so it would run on N/64 CTAs only; split-K GEMM + all-reduce is faster there
                return None
            bn = 128 if ((M + 127) // 128) * ((N + 127) // 128) >= sms else 64
            tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
            need = 2 * (((tiles + self.world_size - 1) // self.world_size) * 128 * bn * 2 * self.world_size + 256 + M * N * 2) + 512
        if tiles > self.max_tiles or need > self.fused_bytes:
            return None
        epi = res = None
        if epilogue is not None:
            residual, norm_w, plus_one = epilogue
            assert residual.dtype == torch.bfloat16 and residual.stride(1) == 1 and residual.shape == (M, N)
            assert norm_w.dtype == torch.bfloat16 and norm_w.is_contiguous()
            qo = torch.empty(M, N, dtype=K.FP8, device=a.device)
            so = K._scale_buf(M, N // 128, a.device)
            ssb = torch.empty(N // bn, (M + 127) // 128 * 128, dtype=torch.float32, device=a.device)
            epi = K._Epilogue()
            epi.mode = 2
            epi.q_out, epi.ldq, epi.s_out, epi.s_ld = qo.data_ptr(), N, so.data_ptr(), so.stride(1)
            epi.residual, epi.ldr, epi.norm_w, epi.norm_plus_one = residual.data_ptr(), residual.stride(0), norm_w.data_ptr(), 1 if plus_one else 0
            epi.ss_out, epi.ss_out_ld = ssb.data_ptr(), ssb.stride(0)
            res = (qo, so, (ssb, N // bn))
        off = _sz(0)
        rc = self.lib.atlas_gemm_allreduce(kind, a.data_ptr(), b.data_ptr(), K._ptr(a_scale),
                                           a_scale.stride(1) if a_scale is not None else 0, K._ptr(b_scale),
                                           b_scale.shape[1] if b_scale is not None else 0, M, N, Kd, a.stride(0), b.stride(0),
                                           bn, self.fdata_arr, self.fflag_arr, self.rank, self.world_size,
                                           self.fstate.data_ptr(), self.fused_bytes, self.max_tiles, C.byref(off), sms,
                                           self.wait_cycles, K._status_ptr[self.dev_index], K._stream(),
                                           1 if oneshot else 0, K._ptr(out), N, splits, K._ptr(ws), K._ptr(cnt),
                                           C.cast(C.byref(epi), _vp) if epi is not None else None)
        K._check(rc, "gemm_allreduce")
        self.calls["gemm_allreduce"] += 1
        if oneshot:
            self.calls["gemm_allreduce_oneshot"] += 1
            return res if epilogue is not None else out
        return _device_view(self._fdata + off.value, (M, N), torch.bfloat16, self.device)

    def seq_parallel(self, tokens: int, hidden: int):
        """The sequence-parallel area (``parallel/seqpar.py``) sized for at least ``tokens`` rows of width ``hidden``:
        allocated symmetrically on every rank and mapped over CUDA IPC on first use (a collective call: every rank
        reaches it with the same arguments).  Returns None when the shape is not covered."""
        self._guard()
        if hidden % 256 or hidden > 16384 or self.world_size > 8:
            return None
        sp = self._sp_areas.get(hidden)
        if sp is not None and sp.t_pad >= tokens:
            return sp
        from .seqpar import SeqParallelArea
        cap = max(tokens, self.sp_min_capacity)
        new = SeqParallelArea(self.rank, self.world_size, cap, hidden, self.device, self.wait_cycles)
        torch.cuda.synchronize(self.device)          # nobody may still be inside kernels that use the old area
        self.base.barrier()
        base = self._alloc(new.nbytes)
        new.adopt(base)
        self._sp_mem.append(base)
        handles = [None] * self.world_size
        self.base.dist.all_gather_object(handles, self._export(base), group=self.base.group)
        new.connect([base if r == self.rank else self._open(h) for r, h in enumerate(handles)])
        self.base.barrier()
        self._sp_areas[hidden] = new
        return new

    # everything else: the bootstrap backend
    def all_reduce_async(self, t):
        """Large messages only (the caller overlaps them with compute): NCCL on its own stream."""
        self._guard()
        self.calls["fallback"] += 1
        return self.base.all_reduce_async(t)

    def all_gather(self, t, dim=0): return self.base.all_gather(t, dim)
    def reduce_scatter(self, t, dim=0): return self.base.reduce_scatter(t, dim)
    def broadcast(self, t, src=0): return self.base.broadcast(t, src)
    def all_to_all(self, parts): return self.base.all_to_all(parts)
    def barrier(self): return self.base.barrier()
    def broadcast_object(self, obj, src=0): return self.base.broadcast_object(obj, src)


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier for memory this module allocated itself."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": tuple(shape), "typestr": typestr, "version": 2,
                                         "strides": None}


def _device_view(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    """A torch tensor aliasing raw device memory (bf16 goes through int16, which the interface can describe)."""
    if dtype == torch.bfloat16:
        return torch.as_tensor(_RawCuda(ptr, shape, "<i2"), device=device).view(torch.bfloat16)
    raise ValueError(dtype)
