"""SwiGLU feed-forward: fused gate|up GEMM -> SiLU*mul (+FP8 quant) -> row-parallel down GEMM.

Under tensor parallelism gate/up are column-parallel and down is row-parallel with its reduction
fused into the GEMM epilogue.  (The reference replicates dense FFN weights across TP ranks,
``crates/spark-model/src/layers/dense_ffn*``; sharding them is this engine's choice.)
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import Act, LinearWeight
from ..lora import add_delta
from .common import ParallelCtx, make_weight, randn_weight, shard_cols, shard_rows


class DenseMLP:
    def __init__(self, cfg: ModelConfig, pctx: ParallelCtx, quant_kind: str, intermediate: Optional[int] = None,
                 shard: bool = True, activation: Optional[str] = None):
        self.cfg, self.pctx, self.quant_kind = cfg, pctx, quant_kind
        # "silu_glu": gate|up GEMM -> silu(gate) * up; "relu2": a single up GEMM -> relu(up)^2 (Nemotron-H)
        self.activation = activation or getattr(cfg, "mlp_activation", "silu_glu")
        self.inter = intermediate or cfg.intermediate_size
        self.shard = shard and pctx.tp_size > 1 and self.inter % (pctx.tp_size * 128) == 0
        self.gate_up: Optional[LinearWeight] = None
        self.down: Optional[LinearWeight] = None
        self.lora = None                    # lora.LoraSet shared by the model's layers
        self.lora_prefix = ""               # e.g. "layers.3.mlp."

    def load(self, gate: Optional[torch.Tensor], up: torch.Tensor, down: torch.Tensor) -> None:
        tp, r = (self.pctx.tp_size, self.pctx.tp_rank) if self.shard else (1, 0)
        if self.activation == "relu2":
            gu = shard_rows(up, r, tp)
        else:
            gu = torch.cat([shard_rows(gate, r, tp), shard_rows(up, r, tp)], 0)
        self.gate_up = make_weight(gu, self.quant_kind)
        self.down = make_weight(shard_cols(down, r, tp).contiguous(), self.quant_kind)

    def init_random(self, gen, std, dtype, device) -> None:
        h = self.cfg.hidden_size
        self.load(randn_weight(gen, self.inter, h, std, dtype, device),
                  randn_weight(gen, self.inter, h, std, dtype, device),
                  randn_weight(gen, h, self.inter, std, dtype, device))

    def hidden_act(self, act: Act) -> Act:
        """gate|up GEMM + SiLU * mul: the input of the down projection (no adapters)."""
        if self.activation == "gelu_tanh_glu":
            return ops.glu_act(ops.linear(act, self.gate_up), self.down.kind == "fp8_block", "gelu_tanh")
        if self.down.kind == "fp8_block" and ops.swiglu_fusable(act, self.gate_up):
            return ops.linear_swiglu(act, self.gate_up)
        return ops.silu_mul_act(ops.linear(act, self.gate_up), want_fp8=self.down.kind == "fp8_block")

    def _relu2(self, act: Act, reduce: bool) -> torch.Tensor:
        u = ops.linear(act, self.gate_up)
        a = ops.relu_squared(u)
        return self.pctx.row_parallel_linear(a, self.down) if (self.shard and reduce) else ops.linear(a, self.down)

    def forward(self, act: Act, reduce: bool = True, batch=None) -> torch.Tensor:
        if self.activation == "relu2":
            return self._relu2(act, reduce)
        use_lora = self.lora is not None and batch is not None and batch.adapter_rows is not None and self.lora_prefix
        if self.activation == "gelu_tanh_glu" and not use_lora:
            a = self.hidden_act(act)
            return self.pctx.row_parallel_linear(a, self.down) if (self.shard and reduce) else ops.linear(a, self.down)
        if not use_lora and self.down.kind == "fp8_block" and ops.swiglu_fusable(act, self.gate_up):
            a = ops.linear_swiglu(act, self.gate_up)
            return self.pctx.row_parallel_linear(a, self.down) if (self.shard and reduce) else ops.linear(a, self.down)
        gu = ops.linear(act, self.gate_up)
        if use_lora:
            xin, half = act.plain(), gu.shape[1] // 2
            add_delta(gu, self.lora, self.lora_prefix + "gate_proj", xin, batch, 0, half)
            add_delta(gu, self.lora, self.lora_prefix + "up_proj", xin, batch, half, half)
        if self.activation == "gelu_tanh_glu":
            a = ops.glu_act(gu, False, "gelu_tanh")
        else:
            a = ops.silu_mul_act(gu, want_fp8=self.down.kind == "fp8_block" and not use_lora)
        if use_lora:
            # with a sharded FFN this rank's columns of A give a partial delta: add it before the group reduction
            y = ops.linear(a, self.down)
            add_delta(y, self.lora, self.lora_prefix + "down_proj", a.plain(), batch)
            return self.pctx.all_reduce(y) if (self.shard and reduce) else y
        if self.shard and reduce:
            return self.pctx.row_parallel_linear(a, self.down)
        return ops.linear(a, self.down)
