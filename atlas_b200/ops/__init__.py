"""Op front-end: every call goes to the sm_100a kernel library when the tensors live on a GPU and to
the plain-PyTorch restatement (``ops.reference``) otherwise.

On a machine with a GPU the kernel library is mandatory: importing this package there without a
built ``libatlas_b200_kernels.so`` raises instead of silently running eager PyTorch.
"""
from __future__ import annotations

from dataclasses import dataclass
import os
from typing import List, Optional, Tuple

import torch

from .. import quant as Q
from . import reference as ref

_cuda = None
FORCE_REFERENCE = False     # run the plain-PyTorch restatement even for GPU tensors (oracle for end-to-end tests)


def on_gpu(t: torch.Tensor) -> bool:
    """True when ``t`` should go to the sm_100a kernels."""
    return t.is_cuda and not FORCE_REFERENCE


def cuda_ops():
    """The ctypes binding module for the kernel library (loaded on first GPU use)."""
    global _cuda
    if _cuda is None:
        from . import cuda as _c
        _c.load()
        _cuda = _c
    return _cuda


# ----------------------------------------------------------------------------- weights / activations
@dataclass
class LinearWeight:
    """One (possibly quantized) ``[N,K]`` projection.

    kind ``dense``: ``weight [N,K]`` in the model dtype.
    kind ``fp8_block``: ``weight [N,K]`` e4m3, ``scale [ceil(N/128), ceil(K/128)]`` fp32.
    kind ``nvfp4``: ``weight [N,K/2]`` packed E2M1, ``scale [N,K/16]`` e4m3, ``gscale`` fp32, ``[1]`` or one per output row ``[N]``.
    """
    kind: str
    weight: torch.Tensor
    scale: Optional[torch.Tensor] = None
    gscale: Optional[torch.Tensor] = None
    bias: Optional[torch.Tensor] = None
    _dense_cache: Optional[torch.Tensor] = None

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @property
    def in_features(self) -> int:
        return self.weight.shape[1] * (2 if self.kind == "nvfp4" else 1)

    def dequantized(self) -> torch.Tensor:
        if self.kind == "dense":
            return self.weight
        if self.kind == "fp8_block":
            return Q.dequantize_fp8_block(self.weight, self.scale)
        return Q.dequantize_nvfp4(self.weight, self.scale, self.gscale)

    @staticmethod
    def from_dense(w: torch.Tensor, kind: str, bias=None) -> "LinearWeight":
        if kind in ("dense", "none"):
            return LinearWeight("dense", w.contiguous(), bias=bias)
        if kind == "fp8_block":
            q, s = Q.quantize_fp8_block(w)
            return LinearWeight("fp8_block", q, s, bias=bias)
        if kind == "nvfp4":
            p, s, g = Q.quantize_nvfp4(w)
            return LinearWeight("nvfp4", p, s, g, bias=bias)
        raise ValueError(kind)


@dataclass
class Act:
    """Activation handle: plain ``x [T,K]`` and/or its FP8 group-quantized form ``(q, s)``."""
    x: Optional[torch.Tensor] = None
    q: Optional[torch.Tensor] = None
    s: Optional[torch.Tensor] = None
    dtype: Optional[torch.dtype] = None      # dtype of the tensor the quantised form was made from
    # rows still arriving from other ranks (sequence-parallel all-gather): (flags address, epoch address, wait cycles);
    # the consuming GEMM polls the flags tile by tile (parallel/seqpar.py)
    ready: Optional[tuple] = None
    # deferred RMSNorm factor: ``(q, s)`` hold ``residual * norm_weight`` and every row still has to be multiplied by
    # rsqrt(sum over parts of sums[part, row] / H + eps); tuple ``(sums [parts, rows_pad] fp32, parts, H, eps)``.  The
    # factor commutes with a linear layer, so the consuming GEMM applies it to its output rows.
    row_ss: Optional[tuple] = None

    @property
    def out_dtype(self) -> torch.dtype:
        return self.x.dtype if self.x is not None else (self.dtype or torch.bfloat16)

    def plain(self) -> torch.Tensor:
        if self.x is None:
            x = (self.q.float().view(self.q.shape[0], -1, 128) * self.s[..., None]).view(self.q.shape)
            if self.row_ss is not None:
                sums, parts, h, eps = self.row_ss
                x = x * torch.rsqrt(sums[:parts, :x.shape[0]].sum(0) / h + eps)[:, None]
            self.x = x.to(self.out_dtype)
        return self.x

    def fp8(self) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.q is None:
            self.q, self.s = quant_fp8(self.x)
        return self.q, self.s


# ----------------------------------------------------------------------------- elementwise / norm
def quant_fp8(x: torch.Tensor, group: int = 128):
    if on_gpu(x):
        return cuda_ops().quant_fp8(x, group)
    return Q.per_token_group_quant_fp8(x, group)


def rmsnorm(x, w, eps, residual=None, plus_one=False):
    if on_gpu(x):
        return cuda_ops().rmsnorm(x, w, eps, residual, plus_one, quant=False)
    return ref.rmsnorm(x, w, eps, residual, plus_one)


def rmsnorm_act(x, w, eps, residual=None, plus_one=False, want_fp8=False) -> Tuple[Act, Optional[torch.Tensor]]:
    """Residual add + RMSNorm, emitting FP8 group-quantized activations when the consumer is an FP8 GEMM."""
    if want_fp8 and x.shape[-1] % 128 == 0:
        if on_gpu(x):
            q, s, r = cuda_ops().rmsnorm(x, w, eps, residual, plus_one, quant=True)
        else:
            q, s, r = ref.rmsnorm_quant_fp8(x, w, eps, residual, plus_one)
        return Act(q=q, s=s, dtype=x.dtype), r
    y, r = rmsnorm(x, w, eps, residual, plus_one)
    return Act(x=y), r


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """``relu(x) ** 2`` (the activation of Nemotron-H's two-projection MLP)."""
    if on_gpu(x) and x.dtype == torch.bfloat16 and x.stride(-1) == 1:
        return cuda_ops().relu_squared(x)
    return torch.relu(x).square()


def glu_act(gate_up: torch.Tensor, want_fp8=False, kind: str = "silu") -> Act:
    """``act(gate) * up`` with ``kind`` in {silu, gelu_tanh}."""
    if kind == "silu":
        return silu_mul_act(gate_up, want_fp8)
    inter = gate_up.shape[-1] // 2
    gpu = on_gpu(gate_up) and gate_up.dtype == torch.bfloat16
    if want_fp8 and inter % 128 == 0:
        if gpu:
            q, s = cuda_ops().gelu_tanh_mul(gate_up, quant=True)
        else:
            q, s = Q.per_token_group_quant_fp8(ref.gelu_tanh_mul(gate_up), 128)
        return Act(q=q, s=s, dtype=gate_up.dtype)
    return Act(x=cuda_ops().gelu_tanh_mul(gate_up) if gpu else ref.gelu_tanh_mul(gate_up))


def silu_mul_act(gate_up: torch.Tensor, want_fp8=False) -> Act:
    inter = gate_up.shape[-1] // 2
    if want_fp8 and inter % 128 == 0:
        if on_gpu(gate_up):
            q, s = cuda_ops().silu_mul(gate_up, quant=True)
        else:
            q, s = ref.silu_mul_quant_fp8(gate_up)
        return Act(q=q, s=s, dtype=gate_up.dtype)
    if on_gpu(gate_up):
        return Act(x=cuda_ops().silu_mul(gate_up, quant=False))
    return Act(x=ref.silu_mul(gate_up))


# ----------------------------------------------------------------------------- GEMM
def linear(a, w: LinearWeight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = a @ W^T (+ bias)``; ``a`` is a tensor or an :class:`Act`."""
    act = a if isinstance(a, Act) else Act(x=a)
    dev_cuda = on_gpu(act.x if act.x is not None else act.q)
    if w.kind == "fp8_block" and act.row_ss is not None and dev_cuda:
        y = cuda_ops().gemm_fp8_fused(act.q, act.s, w.weight, w.scale, mode=0, out=out, ss_in=act.row_ss, ready=act.ready)
    elif w.kind == "fp8_block":
        if act.row_ss is not None:
            act = Act(x=act.plain())
        q, s = act.fp8()
        if dev_cuda:
            y = cuda_ops().gemm_fp8_block(q, s, w.weight, w.scale, out=out, ready=act.ready)
        else:
            y = Q.fp8_block_gemm_ref(q, s, w.weight, w.scale, out_dtype=act.out_dtype)
    elif w.kind == "nvfp4":
        x = act.plain()
        w4a4 = NVFP4_ACTIVATIONS and x.shape[-1] % 64 == 0
        if dev_cuda and w4a4:
            from . import cuda_fp4
            y = cuda_fp4.linear_w4a4(x, w, out=out)
        elif dev_cuda:
            y = cuda_ops().gemm_nvfp4(x, w.weight, w.scale, w.gscale, out=out)
        elif w4a4:
            y = (ref.quant_nvfp4_rowwise(x) @ w.dequantized().t()).to(x.dtype)
        else:
            y = (x.float() @ w.dequantized().t()).to(x.dtype)
    else:
        x = act.plain()
        if dev_cuda and x.dtype == torch.bfloat16 and w.weight.dtype == torch.bfloat16:
            y = cuda_ops().gemm_bf16(x, w.weight, out=out)
        else:
            y = torch.nn.functional.linear(x, w.weight)
    if w.bias is not None:
        y = y + w.bias
    return y


# NVFP4 weights: quantise the activations to NVFP4 too and run the block-scaled FP4 x FP4 tensor-core GEMM (what an
# "NVFP4" ModelOpt checkpoint is calibrated for); off = weight-only (activations stay bf16)
NVFP4_ACTIVATIONS = os.environ.get("ATLAS_NVFP4_W4A4", "0") == "1"

FUSED_EPILOGUES = True      # tests switch this off to compare against the unfused kernel sequence


def swiglu_fusable(a, w: LinearWeight) -> bool:
    """The gate|up GEMM can apply SiLU * mul and the FP8 quantisation of its output in its own epilogue."""
    act = a if isinstance(a, Act) else Act(x=a)
    probe = act.x if act.x is not None else act.q
    return (FUSED_EPILOGUES and on_gpu(probe) and w.kind == "fp8_block" and w.bias is None and w.weight.shape[0] % 256 == 0
            and (w.weight.shape[0] // 2) % 128 == 0)


def linear_swiglu(a, w: LinearWeight) -> Act:
    """``silu(gate) * up`` of the stacked gate|up projection as FP8 group-quantised activations (one kernel)."""
    act = a if isinstance(a, Act) else Act(x=a)
    if act.row_ss is None:
        q, s = act.fp8()
    else:
        q, s = act.q, act.s
    qo, so = cuda_ops().gemm_fp8_fused(q, s, w.weight, w.scale, mode=1, ss_in=act.row_ss, ready=act.ready)
    return Act(q=qo, s=so, dtype=act.out_dtype)


def residual_norm_fusable(residual: torch.Tensor, w: LinearWeight) -> bool:
    """The projection ``w`` can add its output to ``residual`` and emit the normalised FP8 activations of the sum in its
    own epilogue.  (The projection's input never carries a deferred 1/rms factor: it is an attention output or an
    activation product, not a norm output.)"""
    return (FUSED_EPILOGUES and on_gpu(residual) and w.kind == "fp8_block" and w.bias is None and w.weight.shape[0] % 128 == 0
            and residual.dtype == torch.bfloat16 and residual.is_contiguous())


def linear_residual_norm(a, w: LinearWeight, residual: torch.Tensor, norm_w: torch.Tensor, eps: float, plus_one: bool):
    """``residual += a @ W^T`` (in place) and the FP8 form of ``residual * norm_w`` with the row's 1/rms factor left to
    the consumer (``Act.row_ss``): projection, residual add, RMSNorm and quantisation in one kernel."""
    act = a if isinstance(a, Act) else Act(x=a)
    q, s = act.fp8()
    qo, so, (sums, parts) = cuda_ops().gemm_fp8_fused(q, s, w.weight, w.scale, mode=2, residual=residual, norm_w=norm_w,
                                                      plus_one=plus_one, ready=act.ready)
    return Act(q=qo, s=so, dtype=residual.dtype, row_ss=(sums, parts, w.weight.shape[0], eps)), residual


# ----------------------------------------------------------------------------- attention
def qk_norm_rope_kv_write(q, k, v, positions, rope_cache, rotary_dim, k_cache, v_cache, slot_mapping,
                          k_scale=1.0, v_scale=1.0, q_norm_w=None, k_norm_w=None, eps=1e-6, norm_plus_one=False, rotate=False):
    """``rotate``: every q / k / v head goes through the orthonormal Walsh-Hadamard transform after RoPE, so the cache
    holds rotated keys and values (the "turbo8" cache: rotation + FP8) and the attention output comes out rotated too
    (``head_rotate`` takes it back)."""
    if on_gpu(q):
        return cuda_ops().qk_norm_rope_kv_write(q, k, v, positions, rope_cache, rotary_dim, k_cache, v_cache,
                                                slot_mapping, k_scale, v_scale, q_norm_w, k_norm_w, eps, norm_plus_one, rotate)
    return ref.qk_norm_rope_kv_write(q, k, v, positions, rope_cache, rotary_dim, k_cache, v_cache, slot_mapping,
                                     k_scale, v_scale, q_norm_w, k_norm_w, eps, norm_plus_one, rotate)


def head_rotate(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard transform along the last (head) dimension of ``x [T, H, D]``; its own inverse."""
    if on_gpu(x) and x.shape[-1] == 128 and x.dtype == torch.bfloat16 and x.stride(2) == 1 and x.stride(1) == 128:
        return cuda_ops().wht_d128(x)
    return ref.head_rotate(x)


def paged_attention(q, k_cache, v_cache, batch, scale, k_scale=1.0, v_scale=1.0, sliding_window=None) -> torch.Tensor:
    """Attention of the step's query rows over the paged cache. ``batch`` is a ``ForwardBatch``."""
    if on_gpu(q):
        return cuda_ops().paged_attention(q, k_cache, v_cache, batch, scale, k_scale, v_scale, sliding_window)
    return ref.paged_attention(q, k_cache, v_cache, batch.block_tables, batch.seq_lens, batch.query_start_loc,
                               scale, k_scale, v_scale, sliding_window)


def paged_attention_fp8_out(q, k_cache, v_cache, batch, scale, k_scale=1.0, v_scale=1.0, sliding_window=None) -> Optional[Act]:
    """Decode attention that hands its output over already group-quantised for an FP8 output projection (one kernel
    less per layer); None when the step / cache / head size is not covered and the caller takes the bf16 path."""
    if not (FUSED_EPILOGUES and on_gpu(q)):
        return None
    r = cuda_ops().paged_attention_q8(q, k_cache, v_cache, batch, scale, k_scale, v_scale, sliding_window)
    return None if r is None else Act(q=r[0], s=r[1], dtype=q.dtype)


# ----------------------------------------------------------------------------- MoE
def moe_route(logits, top_k, norm_topk, scoring="softmax", bias=None, n_group=0, topk_group=0, scale=1.0, hash_table=None,
              token_ids=None):
    if on_gpu(logits):
        return cuda_ops().moe_route(logits, top_k, norm_topk, scoring, bias, n_group, topk_group, scale, hash_table, token_ids)
    return ref.moe_route(logits, top_k, norm_topk, scoring, bias, n_group, topk_group, scale, hash_table, token_ids)


# ----------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, with_value: bool = False):
    if on_gpu(logits):
        return cuda_ops().argmax(logits, with_value)
    idx = ref.argmax_first(logits)
    if with_value:
        return idx, logits.float().gather(-1, idx[:, None])[:, 0]
    return idx


def sample(logits, temperature, top_k, top_p, min_p, uniform):
    if on_gpu(logits):
        return cuda_ops().sample(logits, temperature, top_k, top_p, min_p, uniform)
    return ref.sample(logits, temperature, top_k, top_p, min_p, uniform)


def logit_edits(logits: torch.Tensor, edits: torch.Tensor) -> None:
    """In-place sparse edits of fp32 ``logits [B, V]``.  ``edits`` is an int32 ``[n, 6]`` tensor of records
    ``(row, token, add, rep, sub, flags)`` with the three floats stored as their bit patterns; a (row, token) pair
    appears at most once.  Per record: ``x += add``; ``x = x / rep if x > 0 else x * rep``; ``x -= sub``; bit 0 of
    ``flags`` sets ``x = -inf``."""
    if edits.shape[0] == 0:
        return
    if on_gpu(logits):
        cuda_ops().logit_edits(logits, edits)
        return
    rows, toks = edits[:, 0].long(), edits[:, 1].long()
    add, rep, sub = (edits[:, i].view(torch.float32) for i in (2, 3, 4))
    x = logits[rows, toks] + add
    x = torch.where(rep != 1.0, torch.where(x > 0, x / rep, x * rep), x) - sub
    x = torch.where((edits[:, 5] & 1).bool(), torch.full_like(x, float("-inf")), x)
    logits[rows, toks] = x


def spec_accept(draft: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Greedy draft acceptance: ``draft [B, K]`` (-1 pads), ``target [B, K+1]`` -> accepted draft count per row."""
    if on_gpu(draft):
        return cuda_ops().spec_accept(draft, target)
    B, K = draft.shape
    ok = (draft == target[:, :K]) & (draft >= 0)
    return ok.long().cumprod(1).sum(1).to(torch.int32)
