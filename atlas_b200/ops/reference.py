"""Plain-PyTorch restatement of every fused op the engine uses.

Each function here is (a) the CPU execution path and (b) the oracle that the
sm_100a kernels in ``atlas_b200/csrc`` are tested against.  They are written
for clarity, in fp32, with the same operation order the kernels use.

Layouts
-------
* activations are flattened over tokens: ``[T, ...]`` (continuous batching);
* paged KV cache: ``k_cache, v_cache [num_blocks, block_size, Hkv, D]`` (NHD),
  ``slot_mapping[t] = block * block_size + offset`` (-1 = padding row);
  reference layout: ``kernels/gb10/common/reshape_and_cache.cu:1-20``;
* GDN state per sequence slot: ``h [Hv, Dk, Dv]`` fp32 and a conv window
  ``[C, W-1]`` (reference: ``crates/spark-model/src/model/ssm_pool.rs``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from ..quant import FP8, FP8_MAX, per_token_group_quant_fp8


# ----------------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
            plus_one: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``r = x + residual``; ``y = r * rsqrt(mean(r^2)+eps) * (w | 1+w)``.  Returns ``(y, r)``."""
    dt = x.dtype
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
        new_res = xf.to(dt)
        xf = new_res.float()          # the kernel normalises the rounded residual stream
    else:
        new_res = None
    var = xf.pow(2).mean(-1, keepdim=True)
    wf = w.float() + 1.0 if plus_one else w.float()
    y = (xf * torch.rsqrt(var + eps) * wf).to(dt)
    return y, new_res


def rmsnorm_quant_fp8(x, w, eps, residual=None, plus_one=False, group: int = 128):
    """Fused residual-add + RMSNorm + per-token-group FP8 quant. Returns ``(q, scale, r)``."""
    y, r = rmsnorm(x, w, eps, residual, plus_one)
    q, s = per_token_group_quant_fp8(y, group)
    return q, s, r


def gated_rmsnorm(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``rmsnorm(x) * w * silu(z)`` over the last dim (GDN output norm)."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps) * w.float()
    return (y * F.silu(z.float())).to(x.dtype)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


# ----------------------------------------------------------------------------- rope
def build_rope_cache(rotary_dim: int, max_pos: int, theta: float, scaling: Optional[dict] = None,
                     device="cpu") -> torch.Tensor:
    """``[max_pos, rotary_dim]`` fp32 table: first half cos, second half sin.

    Supports plain, linear, llama3 and YaRN scaling (reference: ``kernels/gb10/common/rope.cu``).
    """
    if rotary_dim <= 0:                  # position-free attention (no rotation)
        return torch.zeros(max_pos, 0, dtype=torch.float32, device=device)
    half = rotary_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / rotary_dim))
    mscale = 1.0
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if kind == "linear":
            inv_freq = inv_freq / factor
        elif kind == "llama3":
            lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = ((orig / wavelen) - lo) / (hi - lo)
            scaled = torch.where(wavelen > orig / lo, inv_freq / factor,
                                 torch.where(wavelen < orig / hi, inv_freq,
                                             (1 - smooth) * inv_freq / factor + smooth * inv_freq))
            inv_freq = scaled
        elif kind == "yarn":
            orig = float(scaling.get("original_max_position_embeddings", 4096))
            beta_fast, beta_slow = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

            def corr(n_rot):
                return (rotary_dim * math.log(orig / (n_rot * 2 * math.pi))) / (2 * math.log(theta))
            low, high = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), rotary_dim - 1)
            ramp = ((torch.arange(half, dtype=torch.float64) - low) / max(high - low, 1e-3)).clamp(0, 1)
            mask = 1 - ramp
            inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask
            get = lambda m: 1.0 if factor <= 1 else 0.1 * m * math.log(factor) + 1.0
            if scaling.get("attention_factor"):
                mscale = float(scaling["attention_factor"])
            elif scaling.get("mscale") and scaling.get("mscale_all_dim"):     # DeepSeek convention: ratio of the two
                mscale = get(float(scaling["mscale"])) / get(float(scaling["mscale_all_dim"]))
            else:
                mscale = get(1.0)
    t = torch.arange(max_pos, dtype=torch.float64)
    freqs = torch.outer(t, inv_freq)
    cache = torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).float()
    return cache.to(device)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """NeoX ("rotate half") rotary embedding on the first ``rotary_dim`` lanes of ``x [T,H,D]``."""
    half = rotary_dim // 2
    cs = cache[positions.long()]
    cos, sin = cs[:, None, :half], cs[:, None, half:]
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:rotary_dim]
    out = xf.clone()
    out[..., :half] = x1 * cos - x2 * sin
    out[..., half:rotary_dim] = x2 * cos + x1 * sin
    return out.to(x.dtype)


def head_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, plus_one: bool) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    wf = w.float() + 1.0 if plus_one else w.float()
    return (xf * torch.rsqrt(var + eps) * wf).to(x.dtype)


_HADAMARD: dict = {}


def hadamard(d: int, device="cpu") -> torch.Tensor:
    """Orthonormal Sylvester (natural-order) Hadamard matrix ``[d, d]``, ``H[i][j] = (-1)^popcount(i & j) / sqrt(d)``."""
    key = (d, str(device))
    if key not in _HADAMARD:
        assert d > 0 and d & (d - 1) == 0, "the Walsh-Hadamard rotation needs a power-of-two head_dim"
        h = torch.ones(1, 1)
        while h.shape[0] < d:
            h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
        _HADAMARD[key] = (h / d ** 0.5).to(device)
    return _HADAMARD[key]


def head_rotate(x: torch.Tensor) -> torch.Tensor:
    return (x.float() @ hadamard(x.shape[-1], x.device)).to(x.dtype)


def qk_norm_rope_kv_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
                          rope_cache: torch.Tensor, rotary_dim: int,
                          k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor,
                          k_scale: float = 1.0, v_scale: float = 1.0,
                          q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None,
                          eps: float = 1e-6, norm_plus_one: bool = False, rotate: bool = False) -> torch.Tensor:
    """Fused (q/k head RMSNorm) + RoPE + (head rotation) + (FP8 quant) + paged cache write.

    ``q [T,Hq,D]``, ``k,v [T,Hkv,D]``.  Returns the roped ``q``; k/v go to the cache at
    ``slot_mapping`` (rows with slot < 0 are skipped).
    """
    if q_norm_w is not None:
        q = head_rmsnorm(q, q_norm_w, eps, norm_plus_one)
        k = head_rmsnorm(k, k_norm_w, eps, norm_plus_one)
    q = apply_rope(q, positions, rope_cache, rotary_dim)
    k = apply_rope(k, positions, rope_cache, rotary_dim)
    if rotate:
        q, k, v = head_rotate(q), head_rotate(k), head_rotate(v)
    nb, bs, hkv, d = k_cache.shape
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    blk, off = slots // bs, slots % bs          # index the logical dims: the cache may be a permuted view
    if k_cache.dtype == FP8:
        k_cache[blk, off] = (k[valid].float() / k_scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
        v_cache[blk, off] = (v[valid].float() / v_scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    else:
        k_cache[blk, off] = k[valid].to(k_cache.dtype)
        v_cache[blk, off] = v[valid].to(v_cache.dtype)
    return q


# ----------------------------------------------------------------------------- attention
def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_tables: torch.Tensor, seq_lens: torch.Tensor, query_start_loc: torch.Tensor,
                    scale: float, k_scale: float = 1.0, v_scale: float = 1.0,
                    sliding_window: Optional[int] = None) -> torch.Tensor:
    """Causal attention of new query rows over the paged cache (prefill chunks and decode alike).

    Sequence ``b`` owns query rows ``query_start_loc[b]:query_start_loc[b+1]``; its last row sits
    at position ``seq_lens[b]-1``.  ``q [T,Hq,D]`` -> ``out [T,Hq,D]``.
    """
    T, Hq, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    G = Hq // Hkv
    out = torch.zeros_like(q)
    qsl = query_start_loc.tolist()
    sl = seq_lens.tolist()
    for b in range(len(sl)):
        q0, q1 = qsl[b], qsl[b + 1]
        ql, L = q1 - q0, sl[b]
        if ql <= 0 or L <= 0:
            continue
        nblk = (L + bs - 1) // bs
        blocks = block_tables[b, :nblk].long()
        kk = k_cache[blocks].reshape(nblk * bs, Hkv, D)[:L].float() * k_scale
        vv = v_cache[blocks].reshape(nblk * bs, Hkv, D)[:L].float() * v_scale
        qq = q[q0:q1].float().view(ql, Hkv, G, D)
        s = torch.einsum("qhgd,khd->hgqk", qq, kk) * scale
        qpos = torch.arange(L - ql, L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        mask = kpos <= qpos
        if sliding_window:
            mask &= kpos > qpos - sliding_window
        s = s.masked_fill(~mask[None, None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgqk,khd->qhgd", p, vv).reshape(ql, Hq, D)
        out[q0:q1] = o.to(q.dtype)
    return out


# ----------------------------------------------------------------------------- activations
def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``[T, 2I]`` (gate | up) -> ``silu(gate) * up`` ``[T, I]``."""
    i = gate_up.shape[-1] // 2
    g, u = gate_up[..., :i].float(), gate_up[..., i:].float()
    return (F.silu(g) * u).to(gate_up.dtype)


def gelu_tanh_mul(gate_up: torch.Tensor) -> torch.Tensor:
    i = gate_up.shape[-1] // 2
    g, u = gate_up[..., :i].float(), gate_up[..., i:].float()
    return (F.gelu(g, approximate="tanh") * u).to(gate_up.dtype)


def silu_mul_quant_fp8(gate_up: torch.Tensor, group: int = 128):
    y = silu_mul(gate_up)
    return per_token_group_quant_fp8(y, group)


# ----------------------------------------------------------------------------- MoE
def quant_nvfp4_rowwise(x: torch.Tensor) -> torch.Tensor:
    """What the W4A4 path's activation quantiser stands for, as an fp32 matrix: per row a second-level scale
    ``g = amax / (6 * 448)``, per 16 values an e4m3 scale factor against ``g``, values rounded to e2m1."""
    from ..quant import E2M1_MAX, _e2m1_lut, _round_to_e2m1_code
    xf = x.float()
    T, K = xf.shape
    amax = xf.abs().amax(-1, keepdim=True)
    g = torch.where(amax > 0, amax / (E2M1_MAX * FP8_MAX), torch.ones_like(amax))
    grp = xf.view(T, K // 16, 16)
    s8 = (grp.abs().amax(-1) / (E2M1_MAX * g)).clamp(max=FP8_MAX).to(FP8).float()
    s = s8 * g
    inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
    codes = _round_to_e2m1_code(grp * inv[..., None])
    vals = _e2m1_lut(x.device)[codes.long()]
    return (vals * s[..., None]).view(T, K)


def route_scores(logits: torch.Tensor, scoring: str) -> torch.Tensor:
    lf = logits.float()
    if scoring == "sigmoid":
        return torch.sigmoid(lf)
    if scoring == "sqrtsoftplus":
        return torch.sqrt(F.softplus(lf))
    return torch.softmax(lf, -1)


def moe_route(logits: torch.Tensor, top_k: int, norm_topk: bool, scoring: str = "softmax", bias: Optional[torch.Tensor] = None,
              n_group: int = 0, topk_group: int = 0, scale: float = 1.0, hash_table: Optional[torch.Tensor] = None,
              token_ids: Optional[torch.Tensor] = None):
    """Router scores -> (weights ``[T,k]`` fp32, expert ids ``[T,k]`` int32); ties pick the lower id.

    ``bias`` biases the SELECTION only (weights come from the unbiased scores).  ``n_group`` / ``topk_group``: a group
    scores the sum of its two best biased scores and only the best ``topk_group`` groups stay eligible.  ``hash_table
    [vocab, k]`` replaces selection by a lookup on ``token_ids``.  ``scale`` multiplies the final weights.
    """
    probs = route_scores(logits, scoring)
    if hash_table is not None:
        ids = hash_table.to(logits.device)[token_ids.long()].long().clamp(0, probs.shape[-1] - 1)
        w = probs.gather(-1, ids)
        if norm_topk:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return w * scale, ids.to(torch.int32)
    sel = probs if bias is None else probs + bias.float()
    if n_group > 1 and 0 < topk_group < n_group:
        T, E = sel.shape
        g = sel.view(T, n_group, E // n_group)
        gs = g.topk(min(2, g.shape[-1]), dim=-1).values.sum(-1)
        keep = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, _topk_low_ties(gs, topk_group), True)
        sel = g.masked_fill(~keep[..., None], float("-inf")).view(T, E)
    ids = _topk_low_ties(sel, top_k)
    w = probs.gather(-1, ids)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return w * scale, ids.to(torch.int32)


def _topk_low_ties(x: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest along the last dim, descending, ties to the lower index (a stable sort gives that)."""
    return torch.sort(x, dim=-1, descending=True, stable=True).indices[..., :k]


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                topk_ids: torch.Tensor, expert_lo: int = 0) -> torch.Tensor:
    """Dense-math MoE over local experts ``[expert_lo, expert_lo+E_local)``.

    ``w13 [E,2I,H]`` (gate rows then up rows), ``w2 [E,H,I]`` already dequantized.
    Tokens routed to non-local experts contribute zero (their owner rank adds them).
    """
    T, H = x.shape
    E = w13.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(E):
        sel = (topk_ids == (e + expert_lo))
        tok = sel.any(-1).nonzero(as_tuple=True)[0]
        if tok.numel() == 0:
            continue
        wgt = (topk_w * sel).sum(-1)[tok]
        h = xf[tok] @ w13[e].float().t()
        i = h.shape[-1] // 2
        a = (F.silu(h[:, :i]) * h[:, i:]).to(x.dtype).float()
        y = a @ w2[e].float().t()
        out.index_add_(0, tok, y * wgt[:, None])
    return out.to(x.dtype)


# ----------------------------------------------------------------------------- Gated DeltaNet
def causal_conv1d(x: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor,
                  bias: Optional[torch.Tensor] = None, activation: bool = True):
    """Depthwise causal conv over one sequence chunk.

    ``x [L,C]``, ``conv_state [C,W-1]`` (previous inputs, oldest first), ``weight [C,W]``.
    Returns ``(y [L,C], new_state [C,W-1])``.
    """
    L, C = x.shape
    W = weight.shape[-1]
    full = torch.cat([conv_state.float().t(), x.float()], dim=0)      # [W-1+L, C]
    win = full.unfold(0, W, 1)                                         # [L, C, W]
    y = (win * weight.float()[None]).sum(-1)
    if bias is not None:
        y = y + bias.float()
    if activation:
        y = F.silu(y)
    new_state = full[-(W - 1):].t().contiguous().to(conv_state.dtype)
    return y.to(x.dtype), new_state


def gdn_gates(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
    """``g = -exp(A_log) * softplus(a + dt_bias)`` (log decay, fp32), ``beta = sigmoid(b)``."""
    g = -A_log.float().exp() * F.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float())


def gdn_recurrent(q, k, v, g, beta, h0: torch.Tensor, scale: Optional[float] = None):
    """Token-by-token gated delta rule over one sequence.

    ``q,k [L,H,Dk]`` (already l2-normalised), ``v [L,H,Dv]``, ``g,beta [L,H]``, ``h0 [H,Dk,Dv]`` fp32.
    ``h_t = exp(g_t) h_{t-1} + k_t (x) ((v_t - h_{t-1}'^T k_t) beta_t)``, ``o_t = h_t^T q_t * scale``.
    Returns ``(o [L,H,Dv], h_L, h_all [L,H,Dk,Dv])``.
    """
    L, H, Dk = q.shape
    scale = scale if scale is not None else Dk ** -0.5
    h = h0.float().clone()
    outs, hs = [], []
    for t in range(L):
        h = h * g[t].float().exp()[:, None, None]
        kt, vt = k[t].float(), v[t].float()
        mem = torch.einsum("hkv,hk->hv", h, kt)
        delta = (vt - mem) * beta[t].float()[:, None]
        h = h + kt[:, :, None] * delta[:, None, :]
        outs.append(torch.einsum("hkv,hk->hv", h, q[t].float() * scale))
        hs.append(h.clone())
    o = torch.stack(outs).to(v.dtype) if L else torch.zeros(0, H, v.shape[-1], dtype=v.dtype, device=v.device)
    return o, h, (torch.stack(hs) if L else h[None][:0])


def gdn_chunked(q, k, v, g, beta, h0: torch.Tensor, chunk: int = 64, scale: Optional[float] = None):
    """Chunk-parallel form of :func:`gdn_recurrent` (WY/UT transform inside a chunk, state pass between).

    Mirrors what the chunked scan kernel computes; used to test that formulation against the
    sequential recurrence.  Reference: ``kernels/gb10/common/gated_delta_rule_fla.cu`` (CHUNK=64).
    """
    L, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = scale if scale is not None else Dk ** -0.5
    h = h0.float().clone()
    out = torch.zeros(L, H, Dv, dtype=torch.float32, device=q.device)
    for c0 in range(0, L, chunk):
        c1 = min(L, c0 + chunk)
        n = c1 - c0
        qc = q[c0:c1].float().transpose(0, 1) * scale       # [H,n,Dk]
        kc = k[c0:c1].float().transpose(0, 1)
        vc = v[c0:c1].float().transpose(0, 1)
        bc = beta[c0:c1].float().transpose(0, 1)            # [H,n]
        gc = g[c0:c1].float().transpose(0, 1).cumsum(-1)    # cumulative log decay inside chunk
        tril = torch.tril(torch.ones(n, n, dtype=torch.bool, device=q.device), -1)
        tril0 = torch.tril(torch.ones(n, n, dtype=torch.bool, device=q.device))
        decay = (gc[:, :, None] - gc[:, None, :]).masked_fill(~tril0, 0.0)   # [H,n,n] log(G_i/G_j), i>=j
        kk = torch.einsum("hik,hjk->hij", kc, kc)
        A = -(kk * decay.exp() * bc[:, :, None]).masked_fill(~tril, 0.0)   # strictly lower
        # (I - A)^{-1} by forward substitution
        Tm = torch.eye(n, device=q.device).expand(H, n, n).clone()
        for i in range(1, n):
            Tm[:, i, :i] = torch.einsum("hj,hjk->hk", A[:, i, :i], Tm[:, :i, :i])
        u = torch.einsum("hij,hjv->hiv", Tm, vc * bc[:, :, None])
        w = torch.einsum("hij,hjk->hik", Tm, kc * (bc * gc.exp())[:, :, None])
        v_new = u - torch.einsum("hik,hkv->hiv", w, h)
        qk = torch.einsum("hik,hjk->hij", qc, kc)
        attn = (qk * decay.exp()).masked_fill(~tril0, 0.0)
        o = torch.einsum("hik,hkv->hiv", qc * gc.exp()[:, :, None], h) + torch.einsum("hij,hjv->hiv", attn, v_new)
        out[c0:c1] = o.transpose(0, 1)
        glast = gc[:, -1]
        h = h * glast.exp()[:, None, None] + torch.einsum(
            "hik,hiv->hkv", kc * (glast[:, None] - gc).exp()[:, :, None], v_new)
    return out.to(v.dtype), h


# ----------------------------------------------------------------------------- sampling
def argmax_first(logits: torch.Tensor) -> torch.Tensor:
    """Greedy argmax; ties resolve to the lowest index (reference: ``sampler.rs:512``)."""
    lf = logits.float()
    mx = lf.max(-1, keepdim=True).values
    idx = torch.arange(lf.shape[-1], device=lf.device).expand_as(lf)
    big = torch.full_like(idx, lf.shape[-1])
    return torch.where(lf == mx, idx, big).min(-1).values.to(torch.int64)


def apply_penalties(logits: torch.Tensor, token_counts: Optional[torch.Tensor], prompt_mask: Optional[torch.Tensor],
                    repetition: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor) -> torch.Tensor:
    """OpenAI presence/frequency penalties over generated counts + HF repetition penalty over seen tokens."""
    lf = logits.float()
    if token_counts is None:
        return lf
    seen = token_counts > 0
    if prompt_mask is not None:
        seen_rep = seen | prompt_mask
    else:
        seen_rep = seen
    rp = repetition[:, None]
    lf = torch.where(seen_rep, torch.where(lf > 0, lf / rp, lf * rp), lf)
    lf = lf - frequency[:, None] * token_counts.float() - presence[:, None] * seen.float()
    return lf


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor) -> torch.Tensor:
    """Temperature / top-k / top-p / min-p sampling with caller-provided uniforms (one per row).

    Rows with ``temperature == 0`` are greedy.  The filter order is top-k, top-p, min-p over the
    temperature-scaled distribution sorted descending (ties by lower id), then inverse-CDF with
    ``uniform[row]``.
    """
    lf = logits.float()
    B, V = lf.shape
    greedy = argmax_first(lf)
    t = temperature.clamp_min(1e-6)[:, None]
    probs = torch.softmax(lf / t, -1)
    sp, si = torch.sort(probs, dim=-1, descending=True, stable=True)
    rank = torch.arange(V, device=lf.device)[None, :]
    k = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k)[:, None]
    keep = rank < k
    csum = sp.cumsum(-1)
    keep &= (csum - sp) < top_p[:, None]
    keep &= sp >= (min_p[:, None] * sp[:, :1])
    keep[:, 0] = True
    sp = torch.where(keep, sp, torch.zeros_like(sp))
    sp = sp / sp.sum(-1, keepdim=True)
    cdf = sp.cumsum(-1)
    pick = (cdf < uniform[:, None] * (1 - 1e-7)).sum(-1).clamp(max=V - 1)
    sampled = si.gather(1, pick[:, None]).squeeze(1)
    return torch.where(temperature <= 0, greedy, sampled)


def spec_verify_greedy(draft_tokens: torch.Tensor, target_argmax: torch.Tensor):
    """Greedy speculative acceptance.

    ``draft_tokens [B,K]`` proposed tokens, ``target_argmax [B,K+1]`` the target's argmax after
    consuming ``[last, d_0..d_{K-1}]``.  Returns ``(num_accepted [B], out_tokens [B,K+1])`` where
    ``out_tokens[:, :n+1]`` are the tokens to emit (accepted drafts then the bonus/correction).
    """
    B, K = draft_tokens.shape
    match = (draft_tokens == target_argmax[:, :K]).to(torch.int64)
    n_acc = match.cumprod(-1).sum(-1)
    return n_acc, target_argmax.clone()


def spec_verify_sample(draft_tokens, draft_probs, target_probs, uniform, resample_uniform):
    """Rejection-sampling acceptance (Leviathan et al.): accept ``d_i`` iff ``u_i < p(d_i)/q(d_i)``;
    on the first rejection resample from ``norm(max(p - q, 0))``; if all accepted sample the bonus from ``p_K``.

    ``draft_probs [B,K,V]``, ``target_probs [B,K+1,V]``, ``uniform [B,K]``, ``resample_uniform [B]``.
    """
    B, K = draft_tokens.shape
    V = target_probs.shape[-1]
    out = torch.zeros(B, K + 1, dtype=torch.int64, device=draft_tokens.device)
    n_acc = torch.zeros(B, dtype=torch.int64, device=draft_tokens.device)
    for b in range(B):
        n = 0
        for i in range(K):
            d = int(draft_tokens[b, i])
            p, qd = float(target_probs[b, i, d]), float(draft_probs[b, i, d])
            if qd > 0 and float(uniform[b, i]) < min(1.0, p / qd):
                out[b, i] = d
                n += 1
            else:
                break
        if n < K:
            resid = (target_probs[b, n].float() - draft_probs[b, n].float()).clamp_min(0)
            if float(resid.sum()) <= 0:
                resid = target_probs[b, n].float()
        else:
            resid = target_probs[b, K].float()
        cdf = (resid / resid.sum()).cumsum(-1)
        out[b, n] = int((cdf < float(resample_uniform[b]) * (1 - 1e-7)).sum().clamp(max=V - 1))
        n_acc[b] = n
    return n_acc, out
