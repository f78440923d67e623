"""Mamba-2 (SSD) mixer with a per-sequence recurrent state slot (Nemotron-H hybrid models).

Per token, with ``H`` heads of ``P`` channels, ``G`` groups and state size ``N``::

    [z | xBC | dt] = in_proj(u)                       z [H*P], xBC [H*P + 2*G*N], dt [H]
    xBC            = silu(causal_conv1d(xBC) + bias)  depth-wise, width 4, state = last 3 inputs
    x, B, C        = split(xBC)                       x [H,P], B [G,N], C [G,N]
    dt             = max(softplus(dt + dt_bias), dt_min);   a = exp(dt * -exp(A_log))
    h[h]           = a * h[h] + dt * x[h] (x) B[g(h)]   state [H,P,N] fp32
    y[h]           = h[h] C[g(h)] + D[h] * x[h]
    out            = out_proj( group_rmsnorm(y * silu(z)) * w )

The state layout (``conv``, ``h``) and the slot / snapshot / write-on-accept protocol are those of the Gated-DeltaNet
mixer, so the scheduler, prefix cache and host tier treat both alike.  Tensor parallelism is head-parallel.

Reference parity: ``crates/spark-model/src/layers/nemotron_mamba2.rs`` (header: norm -> in_proj -> conv1d with bias +
SiLU -> split -> SSM -> gated norm -> out_proj), ``kernels/gb10/common/mamba2_ssm_decode.cu`` / ``mamba2_ssd_chunk.cu``.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..ops import Act, LinearWeight
from .common import ParallelCtx, make_weight, randn_weight, shard_cols


def mamba2_scan_ref(x, dt, a_log, b, c, d_skip, dt_bias, dt_min, h):
    """Sequential fp32 statement of the recurrence.  ``x [T,H,P]``, ``dt [T,H]`` (raw), ``b, c [T,G,N]``,
    ``h [H,P,N]`` (updated copy returned).  Returns ``(y [T,H,P], h)``."""
    T, H, P = x.shape
    G = b.shape[1]
    rep = H // G
    xf, bf, cf = x.float(), b.float().repeat_interleave(rep, 1), c.float().repeat_interleave(rep, 1)
    dtv = torch.clamp(F.softplus(dt.float() + dt_bias.float()), min=dt_min)            # [T,H]
    decay = torch.exp(dtv * -torch.exp(a_log.float()))                                 # [T,H]
    h = h.float().clone()
    ys = []
    for t in range(T):
        h = h * decay[t][:, None, None] + (dtv[t][:, None] * xf[t])[..., None] * bf[t][:, None, :]
        ys.append((h * cf[t][:, None, :]).sum(-1) + d_skip.float()[:, None] * xf[t])
    return torch.stack(ys).to(x.dtype), h


def gated_group_rmsnorm_ref(y, z, w, group: int, eps: float):
    """``rmsnorm_per_group(y * silu(z)) * w`` over the last dimension split into groups of ``group``."""
    v = y.float() * F.silu(z.float())
    g = v.view(*v.shape[:-1], -1, group)
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps)
    return (g.view(v.shape) * w.float()).to(y.dtype)


class Mamba2Mixer:
    def __init__(self, cfg: ModelConfig, layer_idx: int, pctx: ParallelCtx, quant_kind: str):
        self.cfg, self.layer_idx, self.pctx, self.quant_kind = cfg, layer_idx, pctx, quant_kind
        tp = pctx.tp_size
        assert cfg.mamba_num_heads % tp == 0 and cfg.mamba_n_groups % tp == 0, "mamba heads and groups must divide by tp"
        self.h, self.p, self.n = cfg.mamba_num_heads // tp, cfg.mamba_head_dim, cfg.ssm_state_size
        self.g = cfg.mamba_n_groups // tp
        self.d_inner = self.h * self.p
        self.conv_dim = self.d_inner + 2 * self.g * self.n
        self.W = cfg.mamba_conv_kernel
        self.in_proj: Optional[LinearWeight] = None          # rows [z | x | B | C | dt] of this rank
        self.out_proj: Optional[LinearWeight] = None
        self.conv_w = self.conv_b = None                      # [conv_dim, W], [conv_dim]
        self.A_log = self.D = self.dt_bias = self.norm_w = None
        self._pending = None

    # ------------------------------------------------------------------ weights
    def load(self, in_proj: torch.Tensor, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], A_log, D, dt_bias, norm_w,
             out_proj: torch.Tensor) -> None:
        """Full (unsharded) HF tensors: ``in_proj [2*H*P + 2*G*N + H, hidden]`` rows ``[z | x | B | C | dt]``."""
        cfg, tp, r = self.cfg, self.pctx.tp_size, self.pctx.tp_rank
        HP, GN, Hh = cfg.mamba_num_heads * cfg.mamba_head_dim, cfg.mamba_n_groups * cfg.ssm_state_size, cfg.mamba_num_heads
        z, x, b, c, dt = in_proj.split([HP, HP, GN, GN, Hh], 0)
        sl = lambda t, n: t[r * n:(r + 1) * n]
        di, gn = self.d_inner, self.g * self.n
        fused = torch.cat([sl(z, di), sl(x, di), sl(b, gn), sl(c, gn), sl(dt, self.h)], 0)
        self.in_proj = make_weight(fused.contiguous(), self.quant_kind)
        cw = conv_w.reshape(conv_w.shape[0], -1)
        cx, cb_, cc = cw.split([HP, GN, GN], 0)
        self.conv_w = torch.cat([sl(cx, di), sl(cb_, gn), sl(cc, gn)], 0).contiguous()
        if conv_b is not None:
            bx, bb, bc = conv_b.split([HP, GN, GN], 0)
            self.conv_b = torch.cat([sl(bx, di), sl(bb, gn), sl(bc, gn)], 0).contiguous()
        self.A_log, self.D, self.dt_bias = (sl(t, self.h).float().contiguous() for t in (A_log, D, dt_bias))
        self.norm_w = sl(norm_w, di).contiguous()
        self.out_proj = make_weight(shard_cols(out_proj, r, tp).contiguous(), self.quant_kind)

    def init_random(self, gen, std, dtype, device) -> None:
        cfg = self.cfg
        HP, GN, Hh = cfg.mamba_num_heads * cfg.mamba_head_dim, cfg.mamba_n_groups * cfg.ssm_state_size, cfg.mamba_num_heads
        inp = randn_weight(gen, 2 * HP + 2 * GN + Hh, cfg.hidden_size, std, dtype, device)
        conv = randn_weight(gen, HP + 2 * GN, self.W, 0.2, dtype, device)
        cb = torch.zeros(HP + 2 * GN, dtype=dtype, device=device)
        A_log = torch.log(torch.arange(1, Hh + 1, dtype=torch.float32)).to(device)
        self.load(inp, conv, cb, A_log, torch.ones(Hh, device=device), torch.rand(Hh, generator=gen, device=gen.device).to(device),
                  torch.ones(HP, dtype=dtype, device=device), randn_weight(gen, cfg.hidden_size, HP, std, dtype, device))

    # ------------------------------------------------------------------ state
    def alloc_state(self, num_slots: int, device, conv_dtype) -> dict:
        return {"conv": torch.zeros(num_slots, self.conv_dim, self.W - 1, dtype=conv_dtype, device=device),
                "h": torch.zeros(num_slots, self.h, self.p, self.n, dtype=torch.float32, device=device)}

    # ------------------------------------------------------------------ forward
    def forward(self, act: Act, batch, state: dict) -> torch.Tensor:
        proj = ops.linear(act, self.in_proj)
        di, cd = self.d_inner, self.conv_dim
        z, xbc, dt = proj[:, :di], proj[:, di:di + cd], proj[:, di + cd:]
        if batch.spec_verify:
            self._pending = (xbc.clone(), dt.clone(), list(batch.query_lens_host), list(batch.state_slots_host),
                             list(batch.has_state_host))
        if ops.on_gpu(proj):
            y = ops.cuda_ops().mamba2_forward(self, xbc, dt, batch, state, commit=not batch.spec_verify)
        else:
            y = self._forward_ref(xbc, dt, batch.query_lens_host, batch.state_slots_host, batch.has_state_host, state,
                                  commit=not batch.spec_verify, snapshot_plan=batch.snapshot_plan)
        group = self.d_inner // self.g
        if ops.on_gpu(proj) and y.dtype == torch.bfloat16:
            out = ops.cuda_ops().mamba2_gated_norm(y, z, self.norm_w, group, self.cfg.rms_norm_eps)
        else:
            out = gated_group_rmsnorm_ref(y, z, self.norm_w, group, self.cfg.rms_norm_eps)
        return self.pctx.row_parallel_linear(out, self.out_proj)

    def _forward_ref(self, xbc, dt, qlens: List[int], slots: List[int], has_state: List[bool], state: dict, commit: bool,
                     limit: Optional[List[int]] = None, snapshot_plan: Optional[dict] = None) -> torch.Tensor:
        from ..ops import reference as ref
        T = xbc.shape[0]
        out = torch.zeros(T, self.d_inner, dtype=xbc.dtype, device=xbc.device)
        gn = self.g * self.n
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
                y, conv = ref.causal_conv1d(xbc[rows], conv, self.conv_w, bias=self.conv_b)
                x = y[:, :self.d_inner].reshape(m, self.h, self.p)
                b = y[:, self.d_inner:self.d_inner + gn].reshape(m, self.g, self.n)
                c = y[:, self.d_inner + gn:].reshape(m, self.g, self.n)
                o, h = mamba2_scan_ref(x, dt[rows], self.A_log, b, c, self.D, self.dt_bias, self.cfg.mamba_dt_min, h)
                out[rows] = o.reshape(m, self.d_inner)
                if r1 in snap_at:
                    state["conv"][snap_at[r1]] = conv
                    state["h"][snap_at[r1]] = h
                r0 = r1
            if commit:
                state["conv"][slot] = conv
                state["h"][slot] = h
        return out

    def commit(self, num_accepted_rows: List[int], state: dict) -> None:
        """Fold the first ``num_accepted_rows[i]`` stashed rows of each sequence into its state (write-on-accept)."""
        if self._pending is None:
            return
        xbc, dt, qlens, slots, has_state = self._pending
        self._pending = None
        if ops.on_gpu(xbc):
            ops.cuda_ops().mamba2_commit(self, xbc, dt, qlens, slots, has_state, state, num_accepted_rows)
        else:
            self._forward_ref(xbc, dt, qlens, slots, has_state, state, commit=True, limit=num_accepted_rows)
