"""Mixture-of-experts block: router -> top-k -> expert-parallel grouped FFN -> weighted combine (+ shared expert).

Two expert-parallel modes:

* ``alltoall`` (default on GPUs): tokens are dispatched to the rank owning each selected expert,
  run through the grouped expert GEMMs there, and combined back at the source rank with the router
  weights (dispatch and combine are fused with routing / the weighted sum in the kernels).
* ``allreduce``: every rank runs the router on all tokens, computes only its local experts and the
  partial outputs are summed with an all-reduce.  This is what the reference does
  (``crates/spark-model/src/layers/moe/forward.rs:708-710``) and serves as the baseline.

Reference parity: ``crates/spark-model/src/layers/moe/`` (router kinds, shared-expert blend).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import ops, quant as Q
from ..config import ModelConfig
from ..ops import Act, LinearWeight, reference as ref
from .common import ParallelCtx, make_weight, randn_weight
from ..lora import add_delta
from .mlp import DenseMLP


@dataclass
class ExpertWeights:
    """Stacked local experts. ``w13 [E,2I,H]`` (gate rows then up rows), ``w2 [E,H,I]``.

    kind ``dense`` keeps the model dtype; ``fp8_block`` adds ``*_scale [E, ceil(N/128), ceil(K/128)]``;
    ``nvfp4`` stores packed nibbles ``[E,N,K/2]``, e4m3 ``*_scale [E,N,K/16]`` and fp32 ``*_gscale [E]`` (or ``[E,N]``, one per output row).
    """
    kind: str
    w13: torch.Tensor
    w2: torch.Tensor
    w13_scale: Optional[torch.Tensor] = None
    w2_scale: Optional[torch.Tensor] = None
    w13_gscale: Optional[torch.Tensor] = None
    w2_gscale: Optional[torch.Tensor] = None
    _deq: Optional[tuple] = None

    @property
    def num_local(self) -> int:
        return self.w13.shape[0]

    def dequantized_expert(self, e: int):
        """``(w13 [2I,H], w2 [H,I])`` of local expert ``e`` in a floating-point dtype, without expanding the others."""
        if self.kind == "dense":
            return self.w13[e], self.w2[e]
        if self._deq is not None:
            return self._deq[0][e], self._deq[1][e]
        if self.kind == "fp8_block":
            return (Q.dequantize_fp8_block(self.w13[e], self.w13_scale[e]), Q.dequantize_fp8_block(self.w2[e], self.w2_scale[e]))
        return (Q.dequantize_nvfp4(self.w13[e], self.w13_scale[e], self.w13_gscale[e:e + 1]),
                Q.dequantize_nvfp4(self.w2[e], self.w2_scale[e], self.w2_gscale[e:e + 1]))

    def dequantized(self):
        if self.kind == "dense":
            return self.w13, self.w2
        if self._deq is None:
            E = self.num_local
            if self.kind == "fp8_block":
                a = torch.stack([Q.dequantize_fp8_block(self.w13[e], self.w13_scale[e]) for e in range(E)])
                b = torch.stack([Q.dequantize_fp8_block(self.w2[e], self.w2_scale[e]) for e in range(E)])
            else:
                a = torch.stack([Q.dequantize_nvfp4(self.w13[e], self.w13_scale[e], self.w13_gscale[e:e + 1]) for e in range(E)])
                b = torch.stack([Q.dequantize_nvfp4(self.w2[e], self.w2_scale[e], self.w2_gscale[e:e + 1]) for e in range(E)])
            self._deq = (a, b)
        return self._deq

    @staticmethod
    def from_dense(w13: torch.Tensor, w2: torch.Tensor, kind: str) -> "ExpertWeights":
        if kind in ("dense", "none"):
            return ExpertWeights("dense", w13.contiguous(), w2.contiguous())
        E = w13.shape[0]
        if kind == "fp8_block":
            q13, s13 = zip(*[Q.quantize_fp8_block(w13[e]) for e in range(E)])
            q2, s2 = zip(*[Q.quantize_fp8_block(w2[e]) for e in range(E)])
            return ExpertWeights("fp8_block", torch.stack(q13), torch.stack(q2), torch.stack(s13), torch.stack(s2))
        if kind == "nvfp4":
            a = [Q.quantize_nvfp4(w13[e]) for e in range(E)]
            b = [Q.quantize_nvfp4(w2[e]) for e in range(E)]
            return ExpertWeights("nvfp4", torch.stack([x[0] for x in a]), torch.stack([x[0] for x in b]),
                                 torch.stack([x[1] for x in a]), torch.stack([x[1] for x in b]),
                                 torch.cat([x[2] for x in a]), torch.cat([x[2] for x in b]))
        raise ValueError(kind)


class MoE:
    def __init__(self, cfg: ModelConfig, pctx: ParallelCtx, expert_kind: str, dense_kind: str, ep_mode: str = "auto"):
        self.cfg, self.pctx = cfg, pctx
        self.expert_kind, self.dense_kind = expert_kind, dense_kind
        self.top_k = cfg.num_experts_per_tok
        self.e_lo, self.e_hi = cfg.local_expert_range(pctx.ep_rank, pctx.ep_size)
        self.ep_mode = ep_mode
        self.router: Optional[LinearWeight] = None
        self.experts: Optional[ExpertWeights] = None
        self.shared: Optional[DenseMLP] = None
        self.shared_gate: Optional[torch.Tensor] = None
        self.router_bias: Optional[torch.Tensor] = None      # fp32 [E]: selection-only correction (e_score_correction_bias)
        self.hash_table: Optional[torch.Tensor] = None       # int32 [vocab, k]: static token-id -> expert ids
        self.lora = None                    # lora.LoraSet shared by the model's layers
        self.lora_prefix = ""               # e.g. "layers.3.mlp."
        if cfg.shared_expert_intermediate_size:
            self.shared = DenseMLP(cfg, pctx, dense_kind, cfg.shared_expert_intermediate_size, shard=False)

    # ------------------------------------------------------------------ weights
    def load(self, router: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor) -> None:
        """``w13 [E,2I,H]`` / ``w2 [E,H,I]`` are the *global* expert stacks (or already-local stacks)."""
        self.router = LinearWeight("dense", router.contiguous())
        if w13.shape[0] == self.cfg.num_experts and self.pctx.ep_size > 1:
            w13, w2 = w13[self.e_lo:self.e_hi], w2[self.e_lo:self.e_hi]
        self.experts = ExpertWeights.from_dense(w13, w2, self.expert_kind)

    def init_random(self, gen, std, dtype, device) -> None:
        cfg = self.cfg
        h, i = cfg.hidden_size, cfg.moe_intermediate_size
        router = randn_weight(gen, cfg.num_experts, h, std, dtype, device)
        # draw the global stack so every EP layout sees identical experts for a given seed
        n_local = self.e_hi - self.e_lo
        w13_l, w2_l = [], []
        for e in range(cfg.num_experts):
            a = torch.randn(2 * i, h, generator=gen, dtype=torch.float32, device=gen.device) * std
            b = torch.randn(h, i, generator=gen, dtype=torch.float32, device=gen.device) * std
            if self.e_lo <= e < self.e_hi:
                w13_l.append(a.to(device=device, dtype=dtype))
                w2_l.append(b.to(device=device, dtype=dtype))
        assert len(w13_l) == n_local
        self.router = LinearWeight("dense", router)
        if cfg.router_selection_bias:
            self.router_bias = (torch.rand(cfg.num_experts, generator=gen, device=gen.device) * 0.1).to(device)
        self.experts = ExpertWeights.from_dense(torch.stack(w13_l), torch.stack(w2_l), self.expert_kind)
        if self.shared is not None:
            self.shared.init_random(gen, std, dtype, device)
            self.shared_gate = randn_weight(gen, 1, h, std, dtype, device)

    # ------------------------------------------------------------------ forward
    def forward(self, act: Act, token_ids: Optional[torch.Tensor] = None, batch=None) -> torch.Tensor:
        x = act.plain()
        cfg = self.cfg
        logits = ops.linear(x, self.router)
        adapters = self.lora is not None and batch is not None and batch.adapter_rows is not None and bool(self.lora_prefix)
        if adapters:
            add_delta(logits, self.lora, self.lora_prefix + "gate", x, batch)
        topk_w, topk_ids = ops.moe_route(logits, self.top_k, cfg.norm_topk_prob, cfg.router_scoring, self.router_bias,
                                         cfg.router_n_group, cfg.router_topk_group, cfg.routed_scaling_factor,
                                         self.hash_table, token_ids if self.hash_table is not None else None)
        if ops.on_gpu(x):
            y = ops.cuda_ops().moe_forward(x, topk_w, topk_ids, self.experts, self.e_lo, self.pctx, self.ep_mode)
        else:
            y = self._forward_ref(x, topk_w, topk_ids)
        if adapters:
            y = self._adapter_rows_forward(x, y, topk_w, topk_ids, batch.adapter_rows)
        if self.shared is not None:
            s = self.shared.forward(act, reduce=False, batch=batch)
            if (self.shared_gate is not None and ops.on_gpu(x) and x.dtype == torch.bfloat16 and y.dtype == torch.bfloat16
                    and self.shared_gate.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and y.is_contiguous()):
                return ops.cuda_ops().shared_expert_blend(y if y._base is None else y.clone(), s, x, self.shared_gate)
            if self.shared_gate is not None:
                g = torch.sigmoid(x.float() @ self.shared_gate.float().t())
                s = (s.float() * g).to(s.dtype)
            y = y + s
        return y

    def _adapter_rows_forward(self, x, y, topk_w, topk_ids, adapter_rows) -> torch.Tensor:
        """Routed-expert output of the rows whose adapter carries per-expert matrices for this layer, recomputed with
        ``W + scaling * B A`` in every selected local expert and written over those rows of ``y``.  SwiGLU sits between
        the adapted projections, so the update cannot be added to the base output; the base kernels stay as they are
        and only adapter rows pay (one dequantised expert at a time, eager: a step with adapter rows is not captured).
        Every rank sees the same ``adapter_rows``, so the expert-parallel sum below is entered by all or by none.
        Reference behaviour: ``crates/spark-model/src/layers/moe/lora.rs`` (delta folded around the base grouped GEMM,
        base rows skipped)."""
        layer = int(self.lora_prefix.split(".")[1])
        slots = {s: ad for s, ad in self.lora.slots.items() if layer in ad.expert_layers()}
        if not slots:
            return y
        mask = torch.zeros_like(adapter_rows, dtype=torch.bool)
        for s in slots:
            mask |= adapter_rows == s
        rows = mask.nonzero(as_tuple=True)[0]
        if rows.numel() == 0:
            return y
        xr, ids, wts, slot_r = x[rows].float(), topk_ids[rows].long(), topk_w[rows].float(), adapter_rows[rows]
        part = torch.zeros(rows.numel(), x.shape[1], dtype=torch.float32, device=x.device)
        inter = self.cfg.moe_intermediate_size

        def pair(ad, e, leaf):
            w = ad.weights.get(f"{self.lora_prefix}experts.{e}.{leaf}")
            return None if w is None else (w[0].float(), w[1].float(), ad.scaling)

        def low_rank(v, w):
            return 0.0 if w is None else (v @ w[0].t()) @ w[1].t() * w[2]

        for e in ids.unique().tolist():
            if not (self.e_lo <= e < self.e_hi):
                continue                                   # its owner rank adds it
            w13, w2 = self.experts.dequantized_expert(e - self.e_lo)
            hit = ids == e                                 # [R, k]
            for s, ad in slots.items():
                sel = (hit.any(-1) & (slot_r == s)).nonzero(as_tuple=True)[0]
                if sel.numel() == 0:
                    continue
                xe = xr[sel]
                h = xe @ w13.float().t()
                g = h[:, :inter] + low_rank(xe, pair(ad, e, "gate_proj"))
                u = h[:, inter:] + low_rank(xe, pair(ad, e, "up_proj"))
                a = (torch.nn.functional.silu(g) * u).to(x.dtype).float()
                o = a @ w2.float().t() + low_rank(a, pair(ad, e, "down_proj"))
                part.index_add_(0, sel, o * (wts[sel] * hit[sel]).sum(-1, keepdim=True))
        p = self.pctx
        comm = p.ep_comm if p.ep_comm is not None else p.comm
        if p.ep_size > 1 and comm is not None:
            part = comm.all_reduce(part)
        if y._base is not None:
            y = y.clone()                                  # the fused combine returns a view of its reduction area
        y[rows] = part.to(y.dtype)
        return y

    def _forward_ref(self, x, topk_w, topk_ids) -> torch.Tensor:
        w13, w2 = self.experts.dequantized()
        p = self.pctx
        comm = p.ep_comm if p.ep_comm is not None else p.comm
        mode = self.ep_mode if self.ep_mode != "auto" else "allreduce"
        if p.ep_size == 1 or comm is None:
            return ref.moe_experts(x, w13, w2, topk_w, topk_ids, self.e_lo)
        if mode == "allreduce":
            return comm.all_reduce(ref.moe_experts(x, w13, w2, topk_w, topk_ids, self.e_lo))
        return self._forward_alltoall_ref(x, topk_w, topk_ids, w13, w2, comm)

    def _forward_alltoall_ref(self, x, topk_w, topk_ids, w13, w2, comm) -> torch.Tensor:
        """Host-orchestrated dispatch/combine (what the fused kernels do in one pass)."""
        p, cfg = self.pctx, self.cfg
        T, H = x.shape
        bounds = [cfg.local_expert_range(r, p.ep_size) for r in range(p.ep_size)]
        owner = torch.zeros(cfg.num_experts, dtype=torch.long)
        for r, (lo, hi) in enumerate(bounds):
            owner[lo:hi] = r
        dest = owner.to(x.device)[topk_ids.long()]                        # [T,k]
        send_rows, send_meta = [], []
        for r in range(p.ep_size):
            t_idx, k_idx = (dest == r).nonzero(as_tuple=True)
            send_rows.append(x[t_idx].contiguous())
            send_meta.append(torch.stack([t_idx, topk_ids[t_idx, k_idx].long()], 1) if t_idx.numel() else
                             torch.zeros(0, 2, dtype=torch.long, device=x.device))
        recv_rows = comm.all_to_all(send_rows)
        recv_meta = comm.all_to_all(send_meta)
        outs = []
        for rows, meta in zip(recv_rows, recv_meta):
            if rows.shape[0] == 0:
                outs.append(rows)
                continue
            ids = meta[:, 1:2].to(torch.int32)
            ones = torch.ones(rows.shape[0], 1, dtype=torch.float32, device=rows.device)
            outs.append(ref.moe_experts(rows, w13, w2, ones, ids, self.e_lo))
        back = comm.all_to_all(outs)
        y = torch.zeros(T, H, dtype=torch.float32, device=x.device)
        for r in range(p.ep_size):
            t_idx, k_idx = (dest == r).nonzero(as_tuple=True)
            if t_idx.numel():
                y.index_add_(0, t_idx, back[r].float() * topk_w[t_idx, k_idx][:, None])
        return y.to(x.dtype)
