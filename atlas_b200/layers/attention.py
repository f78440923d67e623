"""GQA attention block over the paged KV cache (optionally with q/k head norms and an output gate).

Data flow per step: fused QKV GEMM -> fused (q/k RMSNorm) + RoPE + FP8 quant + paged-cache write ->
paged attention (split-K decode kernel for single-row sequences, tiled prefill kernel for chunks) ->
(sigmoid gate) -> row-parallel output GEMM whose tensor-parallel reduction is fused into its epilogue.

Reference parity: ``crates/spark-model/src/layers/qwen3_attention/`` (decode:
``trait_impl/decode_inner.rs``, prefill: ``trait_impl/prefill_inner.rs``).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import Act, LinearWeight
from ..lora import GATE_SUFFIX, add_delta
from .common import ParallelCtx, make_weight, randn_weight, shard_cols, shard_rows


class Attention:
    def __init__(self, cfg: ModelConfig, layer_idx: int, pctx: ParallelCtx, quant_kind: str):
        self.cfg, self.layer_idx, self.pctx = cfg, layer_idx, pctx
        tp = pctx.tp_size
        assert cfg.num_attention_heads % tp == 0, "query heads must divide by tp"
        self.hq = cfg.num_attention_heads // tp
        self.hkv = max(1, cfg.num_key_value_heads // tp)
        self.kv_rep = max(1, tp // cfg.num_key_value_heads)     # ranks sharing one kv head
        self.d = cfg.head_dim
        self.gated = cfg.attn_output_gate
        self.scale = cfg.attn_scale or self.d ** -0.5
        # models with per-layer attention kinds (Gemma): only "sliding_attention" layers use the window
        kinds = cfg.layer_types if (cfg.family != "hybrid" and cfg.layer_types) else None
        self.local = bool(kinds) and kinds[layer_idx] == "sliding_attention"
        self.window = cfg.sliding_window if (kinds is None or self.local) else None
        self.quant_kind = quant_kind
        self.qkv: Optional[LinearWeight] = None
        self.o: Optional[LinearWeight] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None
        self.lora = None                    # lora.LoraSet shared by the model's layers
        self.selector = None                # kv.sparse_select.BlockSelector: block-selected decode attention (long contexts)
        self.kv_rotate = False              # "turbo8" cache: q / k / v heads Hadamard-rotated before the FP8 cache write

    # ------------------------------------------------------------------ weights
    def _kv_slice(self, w: torch.Tensor) -> torch.Tensor:
        tp, r = self.pctx.tp_size, self.pctx.tp_rank
        if tp == 1:
            return w
        head = (r // self.kv_rep) * self.hkv
        return w[head * self.d:(head + self.hkv) * self.d]

    def load(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor,
             q_norm=None, k_norm=None, qkv_bias=None) -> None:
        """Takes full (unsharded) HF-layout tensors; slices for this rank, fuses, quantizes."""
        cfg, tp, r = self.cfg, self.pctx.tp_size, self.pctx.tp_rank
        if self.gated:   # HF q_proj rows are per head [q(D) | gate(D)]
            qg = q.view(cfg.num_attention_heads, 2, self.d, -1)
            q, gate = qg[:, 0].reshape(-1, q.shape[-1]), qg[:, 1].reshape(-1, q.shape[-1])
        parts = [shard_rows(q, r, tp), self._kv_slice(k), self._kv_slice(v)]
        if self.gated:
            parts.append(shard_rows(gate, r, tp))
        fused = torch.cat(parts, 0)
        self.qkv = make_weight(fused, self.quant_kind, qkv_bias)
        self.o = make_weight(shard_cols(o, r, tp).contiguous(), self.quant_kind)
        self.q_norm, self.k_norm = q_norm, k_norm

    def init_random(self, gen, std, dtype, device) -> None:
        cfg = self.cfg
        h = cfg.hidden_size
        qmul = 2 if self.gated else 1
        q = randn_weight(gen, cfg.num_attention_heads * self.d * qmul, h, std, dtype, device)
        k = randn_weight(gen, cfg.num_key_value_heads * self.d, h, std, dtype, device)
        v = randn_weight(gen, cfg.num_key_value_heads * self.d, h, std, dtype, device)
        o = randn_weight(gen, h, cfg.num_attention_heads * self.d, std, dtype, device)
        qn = kn = None
        if cfg.qk_norm:
            base = 0.0 if cfg.norm_plus_one else 1.0
            qn = torch.full((self.d,), base, dtype=dtype, device=device)
            kn = torch.full((self.d,), base, dtype=dtype, device=device)
        self.load(q, k, v, o, qn, kn)

    # ------------------------------------------------------------------ forward
    def forward(self, act: Act, batch, kv: Tuple[torch.Tensor, torch.Tensor, float, float],
                rope_cache: torch.Tensor) -> torch.Tensor:
        out = self.mix(act, batch, kv, rope_cache)
        if self.lora is not None and batch.adapter_rows is not None:
            # this rank's columns of A give a partial delta: it joins the partial product before the group reduction
            y = ops.linear(out, self.o)
            add_delta(y, self.lora, f"layers.{self.layer_idx}.self_attn.o_proj", out, batch)
            return self.pctx.all_reduce(y)
        return self.pctx.row_parallel_linear(out, self.o)

    def mix(self, act: Act, batch, kv: Tuple[torch.Tensor, torch.Tensor, float, float],
            rope_cache: torch.Tensor):
        """Everything before the output projection: this rank's heads' attention output ``[T, hq * d]`` (a tensor, or an
        ``Act`` holding its FP8 form when the attention kernel quantised it)."""
        cfg = self.cfg
        k_cache, v_cache, k_scale, v_scale = kv
        qkv = ops.linear(act, self.qkv)
        T = qkv.shape[0]
        nq, nkv = self.hq * self.d, self.hkv * self.d
        if self.lora is not None and batch.adapter_rows is not None:
            xin, pre = act.plain(), f"layers.{self.layer_idx}.self_attn."
            add_delta(qkv, self.lora, pre + "q_proj", xin, batch, 0, nq)
            add_delta(qkv, self.lora, pre + "k_proj", xin, batch, nq, nkv)
            add_delta(qkv, self.lora, pre + "v_proj", xin, batch, nq + nkv, nkv)
            if self.gated:
                add_delta(qkv, self.lora, pre + "q_proj" + GATE_SUFFIX, xin, batch, nq + 2 * nkv, nq)
        q = qkv[:, :nq].view(T, self.hq, self.d)
        k = qkv[:, nq:nq + nkv].view(T, self.hkv, self.d)
        v = qkv[:, nq + nkv:nq + 2 * nkv].view(T, self.hkv, self.d)
        rope_pos, rope_cache = batch.rope_inputs(rope_cache, cfg.mrope_section)
        q = ops.qk_norm_rope_kv_write(q, k, v, rope_pos, rope_cache, cfg.rotary_dim, k_cache, v_cache,
                                      batch.slot_mapping, k_scale, v_scale, self.q_norm, self.k_norm,
                                      cfg.rms_norm_eps, cfg.norm_plus_one, rotate=self.kv_rotate)
        if self.selector is not None:
            from ..kv.sparse_select import attend_selected
            self.selector.on_write(self.layer_idx, k_cache, batch, k_scale)
            out = attend_selected(ops.paged_attention, self.selector, self.layer_idx, q, k_cache, v_cache, batch, self.scale,
                                  k_scale, v_scale, self.window)
        else:
            if (self.o.kind == "fp8_block" and not self.gated and self.o.bias is None and not self.kv_rotate
                    and (self.lora is None or batch.adapter_rows is None)):
                a = ops.paged_attention_fp8_out(q, k_cache, v_cache, batch, self.scale, k_scale, v_scale, self.window)
                if a is not None:
                    return a                  # decode step: rows already quantised for the output projection
            out = ops.paged_attention(q, k_cache, v_cache, batch, self.scale, k_scale, v_scale, self.window)
        if self.kv_rotate:
            out = ops.head_rotate(out)        # sum_j p_j (H v_j) = H o, and H is its own inverse
        out = out.reshape(T, nq)
        if self.gated:
            gate = qkv[:, nq + 2 * nkv:]
            if ops.on_gpu(out) and out.dtype == torch.bfloat16 and nq % 8 == 0 and gate.stride(0) % 8 == 0 and gate.data_ptr() % 16 == 0:
                out = ops.cuda_ops().sigmoid_gate_mul(out, gate)          # one kernel, in place
            else:
                out = (out.float() * torch.sigmoid(gate.float())).to(out.dtype)
        return out
