"""Gated DeltaNet (linear-attention) mixer with a per-sequence recurrent state slot.

``h_t = exp(g_t) h_{t-1} + k_t (x) ((v_t - h_{t-1}^T k_t) beta_t)``, ``o_t = h_t^T q_t``; the state
``h [Hv,Dk,Dv]`` is fp32, gates are computed in fp32 from ``A_log`` / ``dt_bias``.

The checkpoint's interleaved ``in_proj_qkvz`` / ``in_proj_ba`` rows are de-interleaved once at load
(rows reordered to ``[q | k | v | z | b | a]``) so the step needs a single GEMM and no shuffle kernel.
Tensor parallelism is head-parallel.  For speculative verification the layer does not commit its
state: it stashes the rows and :meth:`commit` folds the accepted prefix into the state afterwards
(write-on-accept).

Reference parity: ``crates/spark-model/src/layers/qwen3_ssm/`` and
``kernels/gb10/common/{ssm_preprocess,causal_conv1d,gated_delta_rule*}.cu``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import Act, LinearWeight, reference as ref
from .common import ParallelCtx, make_weight, randn_weight, shard_cols


class GatedDeltaNet:
    def __init__(self, cfg: ModelConfig, layer_idx: int, pctx: ParallelCtx, quant_kind: str):
        self.cfg, self.layer_idx, self.pctx, self.quant_kind = cfg, layer_idx, pctx, quant_kind
        tp = pctx.tp_size
        assert cfg.linear_num_key_heads % tp == 0 and cfg.linear_num_value_heads % tp == 0
        self.hk, self.hv = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.kd, self.vd = self.hk * self.dk, self.hv * self.dv
        self.conv_dim = 2 * self.kd + self.vd
        self.W = cfg.linear_conv_kernel_dim
        self.in_proj: Optional[LinearWeight] = None     # rows [q|k|v|z|b|a]
        self.out_proj: Optional[LinearWeight] = None
        self.conv_w: Optional[torch.Tensor] = None      # [conv_dim, W]
        self.A_log = self.dt_bias = self.norm_w = None
        self._pending = None

    # ------------------------------------------------------------------ weights
    def load(self, qkvz: torch.Tensor, ba: torch.Tensor, conv_w: torch.Tensor, dt_bias, A_log, norm_w,
             out_proj: torch.Tensor) -> None:
        """Arguments are the full HF tensors (``conv_w [C,1,W]`` or ``[C,W]``)."""
        cfg, tp, r = self.cfg, self.pctx.tp_size, self.pctx.tp_rank
        HK, HV, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, self.dk, self.dv
        rep = HV // HK
        H = qkvz.shape[-1]
        g = qkvz.view(HK, 2 * dk + 2 * rep * dv, H)
        q, k = g[:, :dk], g[:, dk:2 * dk]
        v, z = g[:, 2 * dk:2 * dk + rep * dv], g[:, 2 * dk + rep * dv:]
        bag = ba.view(HK, 2 * rep, H)
        b, a = bag[:, :rep], bag[:, rep:]
        ks = slice(r * self.hk, (r + 1) * self.hk)           # head-parallel slice
        fused = torch.cat([q[ks].reshape(-1, H), k[ks].reshape(-1, H), v[ks].reshape(-1, H), z[ks].reshape(-1, H),
                           b[ks].reshape(-1, H), a[ks].reshape(-1, H)], 0)
        self.in_proj = make_weight(fused.contiguous(), self.quant_kind)
        cw = conv_w.reshape(conv_w.shape[0], -1)
        KD, VD = HK * dk, HV * dv
        cq, ck, cv = cw[:KD], cw[KD:2 * KD], cw[2 * KD:2 * KD + VD]
        sk = slice(r * self.kd, (r + 1) * self.kd)
        sv = slice(r * self.vd, (r + 1) * self.vd)
        self.conv_w = torch.cat([cq[sk], ck[sk], cv[sv]], 0).contiguous()
        hv = slice(r * self.hv, (r + 1) * self.hv)
        self.dt_bias, self.A_log = dt_bias[hv].float().contiguous(), A_log[hv].float().contiguous()
        self.norm_w = norm_w
        self.out_proj = make_weight(shard_cols(out_proj, r, tp).contiguous(), self.quant_kind)

    def init_random(self, gen, std, dtype, device) -> None:
        cfg = self.cfg
        H = cfg.hidden_size
        KD = cfg.linear_num_key_heads * self.dk
        VD = cfg.linear_num_value_heads * self.dv
        HV = cfg.linear_num_value_heads
        qkvz = randn_weight(gen, 2 * KD + 2 * VD, H, std, dtype, device)
        ba = randn_weight(gen, 2 * HV, H, std, dtype, device)
        conv = randn_weight(gen, 2 * KD + VD, self.W, 0.2, dtype, device)
        dt_bias = torch.rand(HV, generator=gen, device=gen.device).to(device)
        A_log = torch.log(torch.rand(HV, generator=gen, device=gen.device) * 15 + 1).to(device)
        norm_w = torch.ones(self.dv, dtype=dtype, device=device)
        out = randn_weight(gen, H, VD, std, dtype, device)
        self.load(qkvz, ba, conv, dt_bias, A_log, norm_w, out)

    # ------------------------------------------------------------------ state
    def alloc_state(self, num_slots: int, device, conv_dtype) -> dict:
        return {"conv": torch.zeros(num_slots, self.conv_dim, self.W - 1, dtype=conv_dtype, device=device),
                "h": torch.zeros(num_slots, self.hv, self.dk, self.dv, dtype=torch.float32, device=device)}

    # ------------------------------------------------------------------ forward
    def forward(self, act: Act, batch, state: dict) -> torch.Tensor:
        proj = ops.linear(act, self.in_proj)
        c = self.conv_dim
        mixed, z = proj[:, :c], proj[:, c:c + self.vd]
        b, a = proj[:, c + self.vd:c + self.vd + self.hv], proj[:, c + self.vd + self.hv:]
        if batch.spec_verify:
            self._pending = (mixed.clone(), b.clone(), a.clone(), list(batch.query_lens_host), list(batch.state_slots_host),
                             list(batch.has_state_host))
        if ops.on_gpu(proj):
            o = ops.cuda_ops().gdn_forward(self, mixed, a, b, batch, state, commit=not batch.spec_verify)
        else:
            o = self._forward_ref(mixed, a, b, batch.query_lens_host, batch.state_slots_host, batch.has_state_host,
                                  state, commit=not batch.spec_verify, snapshot_plan=batch.snapshot_plan)
        T = o.shape[0]
        y = ref.gated_rmsnorm(o.view(T, self.hv, self.dv), z.reshape(T, self.hv, self.dv), self.norm_w,
                              self.cfg.rms_norm_eps) if not ops.on_gpu(o) else \
            ops.cuda_ops().gated_rmsnorm(o.view(T, self.hv, self.dv), z.reshape(T, self.hv, self.dv), self.norm_w,
                                         self.cfg.rms_norm_eps)
        return self.pctx.row_parallel_linear(y.reshape(T, self.vd), self.out_proj)

    def _forward_ref(self, mixed, a, b, qlens: List[int], slots: List[int], has_state: List[bool], state: dict,
                     commit: bool, limit: Optional[List[int]] = None, snapshot_plan: Optional[dict] = None) -> torch.Tensor:
        T = mixed.shape[0]
        out = torch.zeros(T, self.hv, self.dv, dtype=mixed.dtype, device=mixed.device)
        rep = self.hv // self.hk
        t0 = 0
        for i, (n, slot) in enumerate(zip(qlens, slots)):
            use = n if limit is None else limit[i]
            base = t0
            t0 += n
            if use == 0:
                continue
            conv = state["conv"][slot] if has_state[i] else torch.zeros_like(state["conv"][slot])
            h = state["h"][slot] if has_state[i] else torch.zeros_like(state["h"][slot])
            cuts = sorted(set([r for r, _ in (snapshot_plan or {}).get(i, []) if 0 < r <= use] + [use]))
            snap_at = {r: d for r, d in (snapshot_plan or {}).get(i, [])}
            r0 = 0
            for r1 in cuts:
                rows = slice(base + r0, base + r1)
                m = r1 - r0
                y, conv = ref.causal_conv1d(mixed[rows], conv, self.conv_w)
                q = ref.l2norm(y[:, :self.kd].reshape(m, self.hk, self.dk))
                k = ref.l2norm(y[:, self.kd:2 * self.kd].reshape(m, self.hk, self.dk))
                v = y[:, 2 * self.kd:].reshape(m, self.hv, self.dv)
                if rep > 1:
                    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
                g, beta = ref.gdn_gates(a[rows], b[rows], self.A_log, self.dt_bias)
                if m > 16:
                    o, h = ref.gdn_chunked(q, k, v, g, beta, h)
                else:
                    o, h, _ = ref.gdn_recurrent(q, k, v, g, beta, h)
                out[rows] = o
                if r1 in snap_at:
                    state["conv"][snap_at[r1]] = conv
                    state["h"][snap_at[r1]] = h
                r0 = r1
            if commit:
                state["conv"][slot] = conv
                state["h"][slot] = h
        return out

    def commit(self, num_accepted_rows: List[int], state: dict) -> None:
        """Fold the first ``num_accepted_rows[i]`` stashed rows of each sequence into its state."""
        if self._pending is None:
            return
        mixed, b, a, qlens, slots, has_state = self._pending
        self._pending = None
        if ops.on_gpu(mixed):
            ops.cuda_ops().gdn_commit(self, mixed, a, b, qlens, slots, has_state, state, num_accepted_rows)
        else:
            self._forward_ref(mixed, a, b, qlens, slots, has_state, state, commit=True, limit=num_accepted_rows)
