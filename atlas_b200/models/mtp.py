"""Multi-token-prediction draft head.

``embed(next token) || target hidden -> (norm each) -> fc [2H->H] -> one attention+FFN layer -> norm``,
logits through the target's shared lm_head.  The head owns one extra paged-KV layer, indexed right
after the target's layers, that shares the target's block tables.

Reference parity: ``crates/spark-model/src/layers/mtp_head/`` (``mtp_head.rs`` header,
``forward.rs``, ``propose_chain.rs``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..layers import ParallelCtx
from ..layers.common import make_weight, randn_weight
from ..ops import Act, LinearWeight
from .batch import ForwardBatch


class MTPHead:
    def __init__(self, cfg: ModelConfig, pctx: ParallelCtx, ep_mode: str = "auto"):
        from .decoder import DecoderLayer
        self.cfg, self.pctx = cfg, pctx
        self.layer_idx = cfg.num_hidden_layers          # cache slot of the head's attention layer
        # the head's block is always a full-attention layer
        self.layer = DecoderLayer(cfg, self.layer_idx, pctx, ep_mode, force_attention=True)
        self.fc: Optional[LinearWeight] = None
        self.norm_e = self.norm_h = self.final_norm = None

    def init_random(self, gen, std, dtype, device) -> None:
        h = self.cfg.hidden_size
        base = 0.0 if self.cfg.norm_plus_one else 1.0
        self.fc = make_weight(randn_weight(gen, h, 2 * h, std, dtype, device), "dense")
        self.norm_e = torch.full((h,), base, dtype=dtype, device=device)
        self.norm_h = torch.full((h,), base, dtype=dtype, device=device)
        self.final_norm = torch.full((h,), base, dtype=dtype, device=device)
        self.layer.init_random(gen, std, dtype, device)

    def alloc_cache(self, store, num_blocks, block_size, kv_dtype, device) -> None:
        from .decoder import alloc_kv
        store.kv[self.layer_idx] = alloc_kv(num_blocks, block_size, self.layer.mixer.hkv, self.cfg.head_dim, kv_dtype, device)
        store.kv_scales[self.layer_idx] = (1.0, 1.0)

    @torch.inference_mode()
    def forward(self, batch: ForwardBatch, token_embeds: torch.Tensor, prev_hidden: torch.Tensor, cache,
                rope_cache: torch.Tensor) -> torch.Tensor:
        """``token_embeds [T,H]`` embeddings of the token at position p+1, ``prev_hidden [T,H]`` the target's
        (or the previous draft step's) hidden at position p.  Returns the head's hidden ``[T,H]``."""
        cfg = self.cfg
        e, _ = ops.rmsnorm(token_embeds, self.norm_e, cfg.rms_norm_eps, None, cfg.norm_plus_one)
        h, _ = ops.rmsnorm(prev_hidden, self.norm_h, cfg.rms_norm_eps, None, cfg.norm_plus_one)
        x = ops.linear(torch.cat([e, h], -1), self.fc)
        x, residual = self.layer.forward(x, None, batch, cache, rope_cache)
        y, _ = ops.rmsnorm(x, self.final_norm, cfg.rms_norm_eps, residual, cfg.norm_plus_one)
        return y
