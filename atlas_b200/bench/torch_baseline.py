"""The repository's OWN library baseline for ``bench.py --impl torch-nccl``: the same wave, model shape and precision
class, executed with stock library kernels only — ``torch._scaled_mm`` (cuBLASLt FP8, row-wise scales),
``scaled_dot_product_attention`` (flash), eager elementwise PyTorch and NCCL all-reduce — and no code from
``atlas_b200``'s kernel library, scheduler or engine.

It is NOT the reference implementation (which cannot be built on the box) and is labelled as this repository's own
baseline wherever its numbers appear.  It exists so that a same-box ratio can be computed: what does the hand-written
sm_100a path buy over a straightforward PyTorch + NCCL program on the same GPUs?

Simplifications that favour the baseline: all requests of a wave have the same length, so the KV cache is a dense
``[B, Hkv, S, D]`` bf16 tensor (no paging, no block tables, no scheduler), prompts are prefilled eight at a time, and
decode runs the whole wave as one static batch.
"""
from __future__ import annotations

import math
import time
from typing import List, Tuple

import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn


def _quant_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Row-wise dynamic FP8 quantisation: one scale per row."""
    amax = x.abs().amax(dim=-1, keepdim=True).float().clamp_min(1e-10)
    s = amax / 448.0
    return (x.float() / s).to(FP8), s


class _Linear:
    def __init__(self, w: torch.Tensor):
        q, s = _quant_rows(w)                      # [N, K] fp8, [N, 1]
        self.wq_t = q.t()                          # column-major [K, N] view, as _scaled_mm wants
        self.ws_t = s.t().contiguous()             # [1, N]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        xq, xs = _quant_rows(x)
        return torch._scaled_mm(xq, self.wq_t, scale_a=xs, scale_b=self.ws_t, out_dtype=torch.bfloat16)


def _rms(x, w, eps):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x, cos, sin):
    # x [T, H, D]; neox layout
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


class TorchNcclDecoder:
    """Dense Llama-shaped decoder, tensor parallel over ``world`` ranks (heads / FFN columns sharded, NCCL sums)."""

    def __init__(self, cfg, rank: int, world: int, device, seed: int = 0):
        self.cfg, self.rank, self.world, self.device = cfg, rank, world, device
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
        self.hq, self.hkv = cfg.num_attention_heads // world, max(1, cfg.num_key_value_heads // world)

        def rnd(n, k):
            return (torch.randn(n, k, generator=g, device=device) * 0.02).bfloat16()
        self.embed = rnd(cfg.vocab_size, H)
        self.layers = []
        for _ in range(cfg.num_hidden_layers):
            self.layers.append(dict(
                qkv=_Linear(rnd((self.hq + 2 * self.hkv) * D, H)), o=_Linear(rnd(H, self.hq * D)),
                gu=_Linear(rnd(2 * I // world, H)), down=_Linear(rnd(H, I // world)),
                n1=torch.ones(H, device=device, dtype=torch.bfloat16), n2=torch.ones(H, device=device, dtype=torch.bfloat16)))
        self.final = torch.ones(H, device=device, dtype=torch.bfloat16)
        self.head = rnd(cfg.vocab_size // world if cfg.vocab_size % world == 0 else cfg.vocab_size, H)
        self.vocab_parallel = world > 1 and cfg.vocab_size % world == 0

    def _sum(self, t):
        if self.world > 1:
            torch.distributed.all_reduce(t)
        return t

    def alloc_cache(self, B: int, S: int):
        D = self.cfg.head_dim
        self.k = [torch.zeros(B, self.hkv, S, D, device=self.device, dtype=torch.bfloat16) for _ in self.layers]
        self.v = [torch.zeros(B, self.hkv, S, D, device=self.device, dtype=torch.bfloat16) for _ in self.layers]
        pos = torch.arange(S, device=self.device).float()
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, D, 2, device=self.device).float() / D))
        ang = pos[:, None] * inv[None]
        self.cos, self.sin = ang.cos(), ang.sin()

    @torch.inference_mode()
    def forward(self, ids: torch.Tensor, b0: int, p0: int) -> torch.Tensor:
        """``ids [b, s]`` for sequences ``b0 .. b0+b`` at positions ``p0 .. p0+s``; returns the last position's hidden."""
        cfg = self.cfg
        b, s = ids.shape
        D = cfg.head_dim
        x = self.embed[ids].view(b * s, -1)
        cos, sin = self.cos[p0:p0 + s].repeat(b, 1)[:, None], self.sin[p0:p0 + s].repeat(b, 1)[:, None]
        for li, L in enumerate(self.layers):
            h = _rms(x, L["n1"], cfg.rms_norm_eps)
            qkv = L["qkv"](h)
            q = qkv[:, :self.hq * D].view(b * s, self.hq, D)
            k = qkv[:, self.hq * D:(self.hq + self.hkv) * D].view(b * s, self.hkv, D)
            v = qkv[:, (self.hq + self.hkv) * D:].view(b * s, self.hkv, D)
            q, k = _rope(q, cos, sin), _rope(k, cos, sin)
            self.k[li][b0:b0 + b, :, p0:p0 + s] = k.view(b, s, self.hkv, D).transpose(1, 2)
            self.v[li][b0:b0 + b, :, p0:p0 + s] = v.view(b, s, self.hkv, D).transpose(1, 2)
            qq = q.view(b, s, self.hq, D).transpose(1, 2)
            kk, vv = self.k[li][b0:b0 + b, :, :p0 + s], self.v[li][b0:b0 + b, :, :p0 + s]
            a = F.scaled_dot_product_attention(qq, kk, vv, is_causal=(s > 1 and p0 == 0), enable_gqa=True)
            a = a.transpose(1, 2).reshape(b * s, self.hq * D)
            x = x + self._sum(L["o"](a))
            h = _rms(x, L["n2"], cfg.rms_norm_eps)
            gu = L["gu"](h)
            half = gu.shape[1] // 2
            x = x + self._sum(L["down"](F.silu(gu[:, :half]) * gu[:, half:]))
        x = _rms(x.view(b, s, -1)[:, -1], self.final, cfg.rms_norm_eps)
        return x

    @torch.inference_mode()
    def next_tokens(self, hidden: torch.Tensor) -> torch.Tensor:
        logits = hidden @ self.head.t()
        if self.vocab_parallel:
            val, idx = logits.float().max(-1)
            idx = idx + self.rank * logits.shape[1]
            pair = torch.stack([val.double(), idx.double()], 1)
            allp = [torch.empty_like(pair) for _ in range(self.world)]
            torch.distributed.all_gather(allp, pair)
            allp = torch.stack(allp, 1)
            best = allp[..., 0].argmax(1)
            return allp[torch.arange(allp.shape[0]), best, 1].long()
        return logits.argmax(-1)

    def wave(self, prompts_pinned: torch.Tensor, osl: int, prefill_batch: int = 8) -> Tuple[int, List[float], float]:
        """One wave: ``prompts_pinned [B, isl]`` int64 in pinned host memory.  Returns (output tokens, ttft per
        request in seconds, device-side seconds).  Inputs travel host -> device every call and each step's tokens are
        read back to the host, like a server would."""
        B, isl = prompts_pinned.shape
        t0 = time.perf_counter()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        ttft = [0.0] * B
        cur = torch.empty(B, dtype=torch.long, device=self.device)
        for b0 in range(0, B, prefill_batch):
            ids = prompts_pinned[b0:b0 + prefill_batch].to(self.device, non_blocking=True)
            tok = self.next_tokens(self.forward(ids, b0, 0))
            cur[b0:b0 + ids.shape[0]] = tok
            tok.cpu()
            now = time.perf_counter() - t0
            for i in range(b0, b0 + ids.shape[0]):
                ttft[i] = now
        n_out = B
        for step in range(1, osl):
            cur = self.next_tokens(self.forward(cur.view(B, 1), 0, isl + step - 1))
            cur.cpu()
            n_out += B
        ev1.record()
        ev1.synchronize()
        return n_out, ttft, ev0.elapsed_time(ev1) / 1e3
