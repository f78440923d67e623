"""Multi-head latent attention (DeepSeek-V2/V3 family) over the paged KV cache.

Projections per token, ``H`` heads, latent rank ``R``, head dims ``nope`` / ``rope`` / ``v``::

    q      = q_b( rmsnorm(q_a(x)) )            or q_proj(x)             [H, nope + rope]
    ckv    = kv_a(x)                                                    [R + rope]   (rope part shared by all heads)
    k_nope, v = split( kv_b( rmsnorm(ckv[:R]) ) )                       [H, nope], [H, v]
    k      = [k_nope | rope(ckv[R:])],   q = [q_nope | rope(q_rope)]
    out    = o_proj( softmax(q k^T * scale) v )

The cache holds the EXPANDED per-head keys and values in the layout of the GQA kernels: every head row is padded to
one common width ``D = cfg.head_dim`` (the next supported size >= nope + rope) and ordered ``[rope | nope | 0]`` so
that the rotary part is the leading ``rotary_dim`` columns, which is what the fused rope + cache-write kernel rotates;
values are ``[v | 0]``.  Zero columns add nothing to q.k and the padded value columns are dropped after attention, so
the result equals the unpadded computation.  Checkpoints store the rope columns interleaved (pairs); the loader
reorders those rows of ``q_b`` / ``kv_a`` to the half-split convention of the rope kernel, which leaves q.k unchanged
because both sides get the same permutation.

The latent-cache ("absorbed") decode form, where the cache holds ``R + rope`` values per token and ``kv_b`` is folded
into the query and output projections, needs an attention kernel with a 576-wide key and 512-wide value; it is not
built here.

Reference parity: ``crates/spark-model/src/layers/deepseek_v41/`` (attention front end, q/kv low-rank projections with
their norms), ``kernels/gb10/common/rope_interleaved.cu`` (pair-interleaved rotary convention).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..ops import Act, LinearWeight
from .common import ParallelCtx, make_weight, randn_weight, shard_cols


def deinterleave_rows(w: torch.Tensor, n: int) -> torch.Tensor:
    """Rows ``[x0, y0, x1, y1, ...]`` (pairs) of the last ``n`` -> ``[x0, x1, ..., y0, y1, ...]`` (half split)."""
    idx = torch.cat([torch.arange(0, n, 2), torch.arange(1, n, 2)])
    return w[idx]


def yarn_mscale(scale: float, m: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0


class MLAttention:
    def __init__(self, cfg: ModelConfig, layer_idx: int, pctx: ParallelCtx, quant_kind: str):
        self.cfg, self.layer_idx, self.pctx, self.quant_kind = cfg, layer_idx, pctx, quant_kind
        tp = pctx.tp_size
        assert cfg.num_attention_heads % tp == 0, "heads must divide by tp"
        self.hq = self.hkv = cfg.num_attention_heads // tp
        self.kv_rep = 1
        self.nope, self.rope, self.vd = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.rank, self.q_rank = cfg.kv_lora_rank, cfg.q_lora_rank
        self.d = cfg.head_dim                                  # padded cache width
        assert self.d >= self.nope + self.rope and self.d >= self.vd
        self.gated = False
        self.scale = (self.nope + self.rope) ** -0.5
        rs = cfg.rope_scaling or {}
        if rs.get("rope_type", rs.get("type", "default")) != "default" and rs.get("mscale_all_dim"):
            m = yarn_mscale(float(rs.get("factor", 1.0)), float(rs["mscale_all_dim"]))
            self.scale *= m * m
        self.q_a: Optional[LinearWeight] = None               # [q_rank, hidden] (absent without the low-rank query)
        self.q_a_norm: Optional[torch.Tensor] = None
        self.q_b: Optional[LinearWeight] = None               # [H*(rope+nope), q_rank or hidden], rows [rope | nope] per head
        self.kv_a: Optional[LinearWeight] = None              # [R + rope, hidden]
        self.kv_a_norm: Optional[torch.Tensor] = None
        self.kv_b: Optional[LinearWeight] = None              # [H*(nope+v), R]
        self.o: Optional[LinearWeight] = None
        self.lora = None
        self.q_norm = self.k_norm = None

    # the fused-epilogue paths of the decoder layer look at ``qkv``: the first projection of this block
    @property
    def qkv(self) -> LinearWeight:
        return self.q_a if self.q_a is not None else self.q_b

    # ------------------------------------------------------------------ weights
    def load(self, q_a, q_a_norm, q_b, kv_a, kv_a_norm, kv_b, o, rope_interleaved: bool = True) -> None:
        """Full HF tensors.  ``q_b`` rows per head ``[nope | rope]``; ``kv_a`` rows ``[R | rope]``; ``kv_b`` rows per
        head ``[nope | v]``.  ``q_a`` / ``q_a_norm`` are None when the query has no low-rank factor."""
        cfg, tp, r = self.cfg, self.pctx.tp_size, self.pctx.tp_rank
        H, qd = cfg.num_attention_heads, self.nope + self.rope
        qh = q_b.view(H, qd, -1)[r * self.hq:(r + 1) * self.hq]
        q_rope = qh[:, self.nope:]
        if rope_interleaved:
            q_rope = torch.stack([deinterleave_rows(h, self.rope) for h in q_rope])
        self.q_b = make_weight(torch.cat([q_rope, qh[:, :self.nope]], 1).reshape(self.hq * qd, -1).contiguous(), self.quant_kind)
        k_rope = kv_a[self.rank:]
        if rope_interleaved:
            k_rope = deinterleave_rows(k_rope, self.rope)
        self.kv_a = make_weight(torch.cat([kv_a[:self.rank], k_rope], 0).contiguous(), self.quant_kind)
        kvh = kv_b.view(H, self.nope + self.vd, -1)[r * self.hq:(r + 1) * self.hq]
        self.kv_b = make_weight(kvh.reshape(self.hq * (self.nope + self.vd), -1).contiguous(), self.quant_kind)
        self.q_a = None if q_a is None else make_weight(q_a.contiguous(), self.quant_kind)
        self.q_a_norm, self.kv_a_norm = q_a_norm, kv_a_norm
        self.o = make_weight(shard_cols(o, r, tp).contiguous(), self.quant_kind)

    def init_random(self, gen, std, dtype, device) -> None:
        cfg = self.cfg
        h, H = cfg.hidden_size, cfg.num_attention_heads
        qd = self.nope + self.rope
        q_a = randn_weight(gen, self.q_rank, h, std, dtype, device) if self.q_rank else None
        q_b = randn_weight(gen, H * qd, self.q_rank or h, std, dtype, device)
        kv_a = randn_weight(gen, self.rank + self.rope, h, std, dtype, device)
        kv_b = randn_weight(gen, H * (self.nope + self.vd), self.rank, std, dtype, device)
        o = randn_weight(gen, h, H * self.vd, std, dtype, device)
        ones = lambda n: torch.ones(n, dtype=dtype, device=device)
        self.load(q_a, ones(self.q_rank) if self.q_rank else None, q_b, kv_a, ones(self.rank), kv_b, o)

    # ------------------------------------------------------------------ forward
    def forward(self, act: Act, batch, kv: Tuple[torch.Tensor, torch.Tensor, float, float],
                rope_cache: torch.Tensor) -> torch.Tensor:
        return self.pctx.row_parallel_linear(self.mix(act, batch, kv, rope_cache), self.o)

    def mix(self, act: Act, batch, kv, rope_cache: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        k_cache, v_cache, k_scale, v_scale = kv
        eps = cfg.rms_norm_eps
        if self.q_a is not None:
            qa = ops.linear(act, self.q_a)
            qn, _ = ops.rmsnorm_act(qa, self.q_a_norm, eps, None, False, self.q_b.kind == "fp8_block")
            qf = ops.linear(qn, self.q_b)
        else:
            qf = ops.linear(act, self.q_b)
        ckv = ops.linear(act, self.kv_a)
        T = qf.shape[0]
        cn, _ = ops.rmsnorm_act(ckv[:, :self.rank].contiguous(), self.kv_a_norm, eps, None, False, self.kv_b.kind == "fp8_block")
        kvf = ops.linear(cn, self.kv_b).view(T, self.hq, self.nope + self.vd)
        qd, D = self.nope + self.rope, self.d
        # padded head rows in the cache layout: q, k = [rope | nope | 0], v = [v | 0]
        q = F.pad(qf.view(T, self.hq, qd), (0, D - qd))
        k = torch.zeros(T, self.hq, D, dtype=qf.dtype, device=qf.device)
        k[:, :, :self.rope] = ckv[:, None, self.rank:]
        k[:, :, self.rope:qd] = kvf[:, :, :self.nope]
        v = F.pad(kvf[:, :, self.nope:], (0, D - self.vd))
        q = ops.qk_norm_rope_kv_write(q, k, v, batch.positions, rope_cache, self.rope, k_cache, v_cache, batch.slot_mapping,
                                      k_scale, v_scale, None, None, eps, False)
        out = ops.paged_attention(q, k_cache, v_cache, batch, self.scale, k_scale, v_scale, None)
        return out[:, :, :self.vd].reshape(T, self.hq * self.vd)
