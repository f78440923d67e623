"""Block-diffusion draft model (DFlash): a small Qwen3-style transformer that proposes a whole block of draft tokens
in ONE forward pass.

Conditioning: the residual-stream states of a few target layers (``target_layer_ids``) at every accepted position are
concatenated and projected by one ``fc`` layer into the drafter's width ("context features").  Every drafter layer
derives keys / values for the context positions from these features with its own k / v projections and keeps them in
a paged cache that shares block ids and slot arithmetic with the target's KV cache, so only positions accepted since
the last step have to be added.  A draft block is ``[anchor, MASK, MASK, ...]`` (the anchor is the token the target
sampled last); queries come from the block only, attention runs over the context positions plus the whole block WITHOUT
a causal mask, and the target's output head turns the block's final hidden states into tokens: position ``j >= 1`` of the
block predicts the token at that position.

Bidirectional attention on the causal paged kernels: after the block's keys / values are written to the cache, each
block row is issued as a one-token "decode" sequence whose length covers the context plus the whole block, so every
row sees every block key.

Reference parity: ``crates/spark-model/src/layers/dflash_head.rs`` (module header), ``dflash_head/precompute_ctx_kv.rs``
(context keys / values from the projected target states), ``dflash_head/forward_block.rs`` (one-pass block forward with
non-causal paged attention), ``dflash_head/propose.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..config import ModelConfig
from ..layers import DenseMLP, ParallelCtx
from ..layers.common import make_weight, randn_weight
from ..ops import Act, LinearWeight
from .batch import ForwardBatch


@dataclass
class DFlashConfig:
    hidden_size: int = 2048
    intermediate_size: int = 6144
    num_hidden_layers: int = 8
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    block_len: int = 16                                   # anchor + (block_len - 1) draft positions
    target_layer_ids: List[int] = field(default_factory=lambda: [1, 10, 19, 28, 37])

    def as_model_config(self, target: ModelConfig) -> ModelConfig:
        return ModelConfig(model_type="qwen3", family="dense", vocab_size=target.vocab_size, hidden_size=self.hidden_size,
                           intermediate_size=self.intermediate_size, num_hidden_layers=self.num_hidden_layers,
                           num_attention_heads=self.num_attention_heads, num_key_value_heads=self.num_key_value_heads,
                           head_dim=self.head_dim, rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta, qk_norm=True,
                           max_position_embeddings=target.max_position_embeddings, dtype=target.dtype)


class _DraftLayer:
    def __init__(self, cfg: ModelConfig, pctx: ParallelCtx):
        self.cfg = cfg
        self.hq, self.hkv, self.d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.q: Optional[LinearWeight] = None
        self.kv: Optional[LinearWeight] = None            # rows [k | v]
        self.o: Optional[LinearWeight] = None
        self.q_norm = self.k_norm = self.input_norm = self.post_norm = None
        self.mlp = DenseMLP(cfg, pctx, "dense", shard=False)

    def init_random(self, gen, std, dtype, device) -> None:
        c = self.cfg
        h = c.hidden_size
        self.q = make_weight(randn_weight(gen, self.hq * self.d, h, std, dtype, device), "dense")
        self.kv = make_weight(randn_weight(gen, 2 * self.hkv * self.d, h, std, dtype, device), "dense")
        self.o = make_weight(randn_weight(gen, h, self.hq * self.d, std, dtype, device), "dense")
        ones = lambda n: torch.ones(n, dtype=dtype, device=device)
        self.q_norm, self.k_norm, self.input_norm, self.post_norm = ones(self.d), ones(self.d), ones(h), ones(h)
        self.mlp.init_random(gen, std, dtype, device)


class BlockDiffusionDrafter:
    def __init__(self, dcfg: DFlashConfig, target):
        self.dcfg, self.target = dcfg, target
        if dcfg.hidden_size != target.cfg.hidden_size:
            raise ValueError("the drafter shares the target's embedding and output head: hidden sizes must match")
        self.cfg = dcfg.as_model_config(target.cfg)
        self.device, self.dtype = target.device, target.dtype
        pctx = ParallelCtx()                               # the drafter is small: replicated on every rank
        self.layers = [_DraftLayer(self.cfg, pctx) for _ in range(dcfg.num_hidden_layers)]
        self.fc: Optional[LinearWeight] = None             # [hidden, n_aux * target_hidden]
        self.feat_norm = self.final_norm = None
        self.mask_embed: Optional[torch.Tensor] = None     # [hidden]: the input of a not-yet-known block position
        self.rope_cache: Optional[torch.Tensor] = None
        self.kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.block_size = 16
        self.scale = self.cfg.head_dim ** -0.5

    # ------------------------------------------------------------------ weights / memory
    def init_random(self, seed: int = 1, std: float = 0.02) -> "BlockDiffusionDrafter":
        gen = torch.Generator(device="cuda" if self.device.type == "cuda" else "cpu")
        gen.manual_seed(seed)
        c, t = self.cfg, self.target.cfg
        n_aux = len(self.dcfg.target_layer_ids)
        self.fc = make_weight(randn_weight(gen, c.hidden_size, n_aux * t.hidden_size, std, self.dtype, self.device), "dense")
        ones = lambda n: torch.ones(n, dtype=self.dtype, device=self.device)
        self.feat_norm, self.final_norm = ones(c.hidden_size), ones(c.hidden_size)
        self.mask_embed = randn_weight(gen, 1, c.hidden_size, std, self.dtype, self.device)[0]
        for l in self.layers:
            l.init_random(gen, std, self.dtype, self.device)
        return self

    def load(self, path: str) -> "BlockDiffusionDrafter":
        """Weights from a safetensors directory with the usual decoder naming: ``fc.weight``, ``hidden_norm.weight``,
        ``mask_embed`` (or ``mask_token_id`` in ``config.json``: the target's embedding row is used), ``norm.weight`` and
        ``layers.N.{input_layernorm, post_attention_layernorm, self_attn.{q,k,v,o}_proj, self_attn.{q,k}_norm,
        mlp.{gate,up,down}_proj}`` (an optional ``model.`` prefix is accepted)."""
        import json
        import os
        from ..loader import Checkpoint
        ck = Checkpoint(path)
        pre = "model." if any(k.startswith("model.") for k in ck.keys()) else ""
        get = lambda n: ck.get(pre + n).to(device=self.device, dtype=self.dtype).contiguous()
        self.fc = make_weight(get("fc.weight"), "dense")
        self.feat_norm, self.final_norm = get("hidden_norm.weight"), get("norm.weight")
        if ck.has(pre + "mask_embed"):
            self.mask_embed = get("mask_embed").reshape(-1)
        else:
            with open(os.path.join(path, "config.json")) as f:
                mid = int(json.load(f).get("mask_token_id", 0))
            self.mask_embed = self.target.embed_tokens(torch.tensor([mid], device=self.device))[0].to(self.dtype)
        for i, l in enumerate(self.layers):
            p = f"layers.{i}."
            l.q = make_weight(get(p + "self_attn.q_proj.weight"), "dense")
            l.kv = make_weight(torch.cat([get(p + "self_attn.k_proj.weight"), get(p + "self_attn.v_proj.weight")], 0), "dense")
            l.o = make_weight(get(p + "self_attn.o_proj.weight"), "dense")
            l.q_norm, l.k_norm = get(p + "self_attn.q_norm.weight"), get(p + "self_attn.k_norm.weight")
            l.input_norm, l.post_norm = get(p + "input_layernorm.weight"), get(p + "post_attention_layernorm.weight")
            l.mlp.load(get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight"), get(p + "mlp.down_proj.weight"))
        ck.close()
        return self

    def finalize(self, max_pos: int) -> None:
        from ..ops import reference as ref
        self.rope_cache = ref.build_rope_cache(self.cfg.head_dim, max_pos, self.cfg.rope_theta, None, self.device)

    def alloc_cache(self, num_blocks: int, block_size: int) -> None:
        """Drafter keys / values, 16-bit, same block ids as the target's cache."""
        from .decoder import alloc_kv
        self.block_size = block_size
        for i, l in enumerate(self.layers):
            self.kv[i] = alloc_kv(num_blocks, block_size, l.hkv, l.d, self.dtype if self.dtype != torch.float32 else torch.float32,
                                  self.device)

    # ------------------------------------------------------------------ pieces
    def _norm(self, x, w):
        y, _ = ops.rmsnorm(x, w, self.cfg.rms_norm_eps, None, False)
        return y

    def _write_kv(self, layer_idx: int, feats_or_hidden: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                  q: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """k / v of ``feats_or_hidden`` rows -> k-norm, rotation at ``positions``, paged write at ``slots``.  When ``q`` rows
        are given they are normed and rotated alongside and returned."""
        l = self.layers[layer_idx]
        T = feats_or_hidden.shape[0]
        kv = ops.linear(feats_or_hidden, l.kv)
        k = kv[:, :l.hkv * l.d].reshape(T, l.hkv, l.d)
        v = kv[:, l.hkv * l.d:].reshape(T, l.hkv, l.d)
        if q is None:
            q = torch.zeros(T, l.hq, l.d, dtype=kv.dtype, device=kv.device)       # rotated and dropped
        kc, vc = self.kv[layer_idx]
        return ops.qk_norm_rope_kv_write(q, k, v, positions, self.rope_cache, l.d, kc, vc, slots, 1.0, 1.0, l.q_norm, l.k_norm,
                                         self.cfg.rms_norm_eps, False)

    def context_features(self, aux: Sequence[torch.Tensor]) -> torch.Tensor:
        """``aux``: one ``[T, target_hidden]`` tensor per captured target layer -> ``[T, hidden]`` features."""
        return self._norm(ops.linear(torch.cat(list(aux), -1), self.fc), self.feat_norm)

    def add_context(self, feats: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor) -> None:
        """Keys / values of accepted positions into every layer's cache."""
        for i in range(len(self.layers)):
            self._write_kv(i, feats, positions, slots)

    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.target.embed_tokens(tokens)

    # ------------------------------------------------------------------ one block
    @torch.inference_mode()
    def propose(self, anchors: List[int], ctx_lens: List[int], tables: List[List[int]], num_drafts: int) -> List[List[int]]:
        """Draft ``num_drafts`` tokens for each sequence.  ``anchors[b]`` sits at position ``ctx_lens[b]`` (the context
        cache holds positions ``< ctx_lens[b]``); ``tables[b]`` must cover ``ctx_lens[b] + num_drafts + 1`` positions."""
        B, g = len(anchors), num_drafts + 1
        dev, bs = self.device, self.block_size
        x = self.mask_embed.to(self.dtype).repeat(B * g, 1)
        x[0::g] = self.embed(torch.tensor(anchors, dtype=torch.int64, device=dev)).to(x.dtype)
        pos, slots = [], []
        for b in range(B):
            for j in range(g):
                p = ctx_lens[b] + j
                pos.append(p)
                slots.append(tables[b][p // bs] * bs + p % bs)
        pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
        slot_t = torch.tensor(slots, dtype=torch.int32, device=dev)
        # every block row as a one-token sequence that ends after the whole block: sees context + all block keys
        fb = ForwardBatch.build([[0]] * (B * g), [ctx_lens[b] + g - 1 for b in range(B) for _ in range(g)],
                                [tables[b] for b in range(B) for _ in range(g)], bs, device=dev)
        eps = self.cfg.rms_norm_eps
        residual = None
        for i, l in enumerate(self.layers):
            if residual is None:
                act, _ = ops.rmsnorm_act(x, l.input_norm, eps, None, False, False)
                residual = x
            else:
                act, residual = ops.rmsnorm_act(x, l.input_norm, eps, residual, False, False)
            h = act.plain()
            q = ops.linear(h, l.q).reshape(B * g, l.hq, l.d)
            q = self._write_kv(i, h, pos_t, slot_t, q)
            kc, vc = self.kv[i]
            a = ops.paged_attention(q, kc, vc, fb, self.scale, 1.0, 1.0, None).reshape(B * g, l.hq * l.d)
            o = ops.linear(a, l.o)
            act, residual = ops.rmsnorm_act(o, l.post_norm, eps, residual, False, False)
            x = l.mlp.forward(act, batch=fb)
        y, _ = ops.rmsnorm(x, self.final_norm, eps, residual, False)
        rows = torch.tensor([b * g + j for b in range(B) for j in range(1, g)], dtype=torch.long, device=dev)
        toks = ops.argmax(self.target.compute_logits(y[rows])).view(B, num_drafts).tolist()
        return [[int(t) for t in row] for row in toks]
