"""Generic decoder-only LM assembled from the layer blocks.

One class covers the dense (Llama/Mistral/Qwen2/Qwen3), MoE (Qwen3-MoE) and hybrid
(Qwen3-Next: Gated DeltaNet + gated attention + MoE + MTP head) families; ``ModelConfig`` decides
the mixer and FFN kind of every layer.

Reference parity: ``crates/spark-model/src/model/`` (``TransformerModel``), the decode program in
``model/trait_impl/decode_a2.rs`` and the chunked prefill program in ``model/trait_impl/prefill_b.rs``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..config import ModelConfig
from ..layers import Attention, DenseMLP, GatedDeltaNet, Mamba2Mixer, MLAttention, MoE, ParallelCtx
from ..layers.common import make_weight, randn_weight, shard_rows
from ..ops import Act, LinearWeight, reference as ref
from .batch import ForwardBatch

# tensor-parallel steps with at least this many rows run sequence-parallel (reduce-scatter / all-gather fused into the
# GEMMs); smaller steps keep the replicated residual stream and the fused GEMM + all-reduce
SEQ_PARALLEL_MIN_TOKENS = int(os.environ.get("ATLAS_SP_MIN_TOKENS", "1024"))
# smallest tensor-parallel group whose pure decode steps take the sequence-parallel path (0 = never)
SEQ_PARALLEL_DECODE_MIN_WORLD = int(os.environ.get("ATLAS_SP_DECODE_MIN_WORLD", "0"))

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
           "torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}


def kv_dtype_is_fp8(dtype) -> bool:
    return dtype == torch.float8_e4m3fn


KV_NVFP4 = torch.uint8          # cache dtype marker of the NVFP4 KV cache (packed e2m1 + e4m3 scales, GPU only)


def kv_dtype_is_quantised(dtype) -> bool:
    return dtype == torch.float8_e4m3fn or dtype == KV_NVFP4


def kv_element_bytes(dtype) -> float:
    """Bytes per cached element (NVFP4: half a byte of data plus one scale byte per 16 elements)."""
    return 9.0 / 16.0 if dtype == KV_NVFP4 else float(dtype.itemsize)


def alloc_kv(num_blocks: int, block_size: int, hkv: int, d: int, dtype, device):
    """Paged K and V pools as logical ``[num_blocks, block_size, Hkv, D]`` tensors (the GPU pools are views
    of the kernels' physical layout)."""
    if torch.device(device).type == "cuda" and (kv_dtype_is_quantised(dtype) or dtype == torch.bfloat16):
        return ops.cuda_ops().alloc_kv_cache(num_blocks, block_size, hkv, d, dtype, device)
    if dtype == KV_NVFP4:
        raise ValueError("the NVFP4 KV cache exists on the GPU kernels only")
    shape = (num_blocks, block_size, hkv, d)
    return torch.zeros(shape, dtype=dtype, device=device), torch.zeros(shape, dtype=dtype, device=device)


def torch_dtype(name: str) -> torch.dtype:
    return _DTYPES.get(str(name), torch.bfloat16)


def quant_kinds(cfg: ModelConfig) -> Tuple[str, str]:
    """(kind for dense projections, kind for MoE expert stacks)."""
    m = cfg.quant.method
    if m == "fp8_block":
        return "fp8_block", "fp8_block"
    if m == "nvfp4":
        return ("dense" if cfg.quant.experts_only else "nvfp4"), "nvfp4"
    return "dense", "dense"


@dataclass
class CacheStore:
    """Device memory the model reads/writes across steps: paged KV per attention layer and the
    recurrent-state slot pool per GDN layer."""
    kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)
    kv_scales: Dict[int, Tuple[float, float]] = field(default_factory=dict)
    states: Dict[int, dict] = field(default_factory=dict)
    block_size: int = 16
    num_blocks: int = 0

    def layer_kv(self, i: int):
        k, v = self.kv[i]
        ks, vs = self.kv_scales.get(i, (1.0, 1.0))
        return k, v, ks, vs


class DecoderLayer:
    def __init__(self, cfg: ModelConfig, idx: int, pctx: ParallelCtx, ep_mode: str = "auto",
                 force_attention: bool = False):
        self.cfg, self.idx = cfg, idx
        dense_kind, expert_kind = quant_kinds(cfg)
        self.kind = "attention" if force_attention else cfg.layer_kind(idx)
        attn_cls = MLAttention if cfg.kv_lora_rank > 0 else Attention
        self.mixer = attn_cls(cfg, idx, pctx, dense_kind) if self.kind == "attention" else GatedDeltaNet(cfg, idx, pctx, dense_kind)
        self.is_moe = (cfg.num_experts > 0) if force_attention else cfg.is_moe_layer(idx)
        self.ffn = MoE(cfg, pctx, expert_kind, dense_kind, ep_mode) if self.is_moe else DenseMLP(cfg, pctx, dense_kind)
        self.input_norm: Optional[torch.Tensor] = None
        self.post_norm: Optional[torch.Tensor] = None
        # sandwich norms (Gemma): post_norm normalises the mixer's OUTPUT, pre_ffn_norm the FFN's input, post_ffn_norm
        # the FFN's output; without them post_norm is the FFN's input norm
        self.pre_ffn_norm: Optional[torch.Tensor] = None
        self.post_ffn_norm: Optional[torch.Tensor] = None
        self.rope_override: Optional[torch.Tensor] = None     # rotary table of sliding-window layers with their own base

    def init_random(self, gen, std, dtype, device):
        base = 0.0 if self.cfg.norm_plus_one else 1.0
        self.input_norm = torch.full((self.cfg.hidden_size,), base, dtype=dtype, device=device)
        self.post_norm = torch.full((self.cfg.hidden_size,), base, dtype=dtype, device=device)
        if self.cfg.sandwich_norms:
            self.pre_ffn_norm = torch.full((self.cfg.hidden_size,), base, dtype=dtype, device=device)
            self.post_ffn_norm = torch.full((self.cfg.hidden_size,), base, dtype=dtype, device=device)
        self.mixer.init_random(gen, std, dtype, device)
        self.ffn.init_random(gen, std, dtype, device)

    def _mixer_fp8(self) -> bool:
        w = self.mixer.qkv if self.kind == "attention" else self.mixer.in_proj
        return w.kind == "fp8_block"

    def _ffn_fp8(self) -> bool:
        return (not self.is_moe) and self.ffn.gate_up.kind == "fp8_block"

    def accepts_prenormed(self) -> bool:
        """This layer's input norm may be applied by the previous layer's down projection (deferred 1/rms factor): its
        only consumer of the normalised input is an FP8 linear layer."""
        return (self.kind == "attention" and isinstance(self.mixer, Attention) and self.mixer.qkv.kind == "fp8_block"
                and self.mixer.lora is None and not self.cfg.sandwich_norms)

    def forward(self, x, residual: Optional[torch.Tensor], batch: ForwardBatch, cache: CacheStore,
                rope_cache: torch.Tensor, next_norm: Optional[torch.Tensor] = None):
        """``x`` is the previous layer's output (to be added to ``residual`` and normalised here) or, when that layer
        already did both in its down projection's epilogue, the normalised activations as an ``Act``.  With
        ``next_norm`` (the next layer's input norm weight) this layer may do the same for its successor and return an
        ``Act`` in place of the plain output."""
        cfg = self.cfg
        eps, p1 = cfg.rms_norm_eps, cfg.norm_plus_one
        if self.rope_override is not None:
            rope_cache = self.rope_override
        if isinstance(x, Act):
            act = x
        elif residual is None:
            act, _ = ops.rmsnorm_act(x, self.input_norm, eps, None, p1, self._mixer_fp8())
            residual = x
        else:
            act, residual = ops.rmsnorm_act(x, self.input_norm, eps, residual, p1, self._mixer_fp8())
        if cfg.sandwich_norms:
            h = self.mixer.forward(act, batch, cache.layer_kv(self.idx), rope_cache)
            h, _ = ops.rmsnorm(h, self.post_norm, eps, None, p1)
            act, residual = ops.rmsnorm_act(h, self.pre_ffn_norm, eps, residual, p1, self._ffn_fp8())
            h = self.ffn.forward(act, batch=batch)
            h, _ = ops.rmsnorm(h, self.post_ffn_norm, eps, None, p1)
            return h, residual
        single = self.mixer.pctx.tp_size == 1
        no_lora = batch.adapter_rows is None
        dense_fp8_ffn = self._ffn_fp8() and self.ffn.down.kind == "fp8_block"
        if (self.kind == "attention" and single and no_lora and dense_fp8_ffn
                and ops.residual_norm_fusable(residual, self.mixer.o)):
            # o_proj + residual add + post-attention norm + FP8 quantisation in the projection's epilogue
            out = self.mixer.mix(act, batch, cache.layer_kv(self.idx), rope_cache)
            act, residual = ops.linear_residual_norm(out, self.mixer.o, residual, self.post_norm, eps, p1)
        else:
            fused = None
            tp_fusable = (not single and no_lora and dense_fp8_ffn and isinstance(self.mixer, Attention)
                          and getattr(self.ffn, "shard", False))
            if self.kind == "attention" and tp_fusable:
                # tensor parallel: o_proj + all-reduce + residual add + norm + FP8 quantisation in one kernel (decode-size
                # outputs; larger ones return None before anything is launched)
                out = self.mixer.mix(act, batch, cache.layer_kv(self.idx), rope_cache)
                fused = self.mixer.pctx.row_parallel_residual_norm(out, self.mixer.o, residual, self.post_norm, eps, p1)
                if fused is None:
                    h = self.mixer.pctx.row_parallel_linear(out, self.mixer.o)
            elif self.kind == "attention":
                h = self.mixer.forward(act, batch, cache.layer_kv(self.idx), rope_cache)
            else:
                h = self.mixer.forward(act, batch, cache.states[self.idx])
            if fused is not None:
                act, residual = fused
            else:
                act, residual = ops.rmsnorm_act(h, self.post_norm, eps, residual, p1, self._ffn_fp8())
        if (next_norm is not None and single and no_lora and dense_fp8_ffn
                and ops.residual_norm_fusable(residual, self.ffn.down)):
            # down_proj + residual add + the NEXT layer's input norm + FP8 quantisation in one epilogue
            return ops.linear_residual_norm(self.ffn.hidden_act(act), self.ffn.down, residual, next_norm, eps, p1)
        if (next_norm is not None and not single and no_lora and dense_fp8_ffn and getattr(self.ffn, "shard", False)
                and self.ffn.activation != "relu2" and ops.residual_norm_fusable(residual, self.ffn.down)):
            a = self.ffn.hidden_act(act)
            fused = self.ffn.pctx.row_parallel_residual_norm(a, self.ffn.down, residual, next_norm, eps, p1)
            if fused is not None:
                return fused
            return self.ffn.pctx.row_parallel_linear(a, self.ffn.down), residual
        if self.is_moe:
            hashed = self.ffn.hash_table is not None and batch.input_ids is not None
            h = self.ffn.forward(act, batch.input_ids.to(torch.int32) if hashed else None, batch=batch)
        else:
            h = self.ffn.forward(act, batch=batch)
        return h, residual


class SingleBlock:
    """A pre-norm residual block around ONE module (Nemotron-H): a Mamba-2 mixer, a position-free attention layer or a
    two-projection relu^2 MLP.  Same ``forward`` protocol as :class:`DecoderLayer`: the block's output is added to the
    residual stream by the next block's norm kernel."""

    def __init__(self, cfg: ModelConfig, idx: int, pctx: ParallelCtx):
        self.cfg, self.idx = cfg, idx
        dense_kind, _ = quant_kinds(cfg)
        self.block = cfg.block_types[idx]
        self.kind = cfg.layer_kind(idx)
        self.is_moe = False
        self.mixer = self.ffn = None
        if self.kind == "mamba2":
            self.mixer = Mamba2Mixer(cfg, idx, pctx, dense_kind)
        elif self.kind == "attention":
            self.mixer = Attention(cfg, idx, pctx, dense_kind)
        elif self.block == "mlp":
            self.ffn = DenseMLP(cfg, pctx, dense_kind, activation="relu2")
        else:
            raise ValueError(f"unsupported block type '{self.block}'")
        self.input_norm: Optional[torch.Tensor] = None
        self.post_norm = None

    def init_random(self, gen, std, dtype, device):
        self.input_norm = torch.ones(self.cfg.hidden_size, dtype=dtype, device=device)
        (self.mixer or self.ffn).init_random(gen, std, dtype, device)

    def accepts_prenormed(self) -> bool:
        return False

    def _fp8_in(self) -> bool:
        w = self.mixer.in_proj if self.kind == "mamba2" else (self.mixer.qkv if self.kind == "attention" else self.ffn.gate_up)
        return w.kind == "fp8_block"

    def forward(self, x, residual, batch: ForwardBatch, cache: CacheStore, rope_cache, next_norm=None):
        cfg = self.cfg
        if residual is None:
            act, _ = ops.rmsnorm_act(x, self.input_norm, cfg.rms_norm_eps, None, cfg.norm_plus_one, self._fp8_in())
            residual = x
        else:
            act, residual = ops.rmsnorm_act(x, self.input_norm, cfg.rms_norm_eps, residual, cfg.norm_plus_one, self._fp8_in())
        if self.kind == "mamba2":
            h = self.mixer.forward(act, batch, cache.states[self.idx])
        elif self.kind == "attention":
            h = self.mixer.forward(act, batch, cache.layer_kv(self.idx), rope_cache)
        else:
            h = self.ffn.forward(act, batch=batch)
        return h, residual


class DecoderLM:
    def __init__(self, cfg: ModelConfig, pctx: Optional[ParallelCtx] = None, device="cpu", ep_mode: str = "auto",
                 with_mtp: Optional[bool] = None):
        self.cfg = cfg
        self.pctx = pctx or ParallelCtx()
        self.device = torch.device(device)
        self.dtype = torch_dtype(cfg.dtype)
        if cfg.block_types:
            self.layers = [SingleBlock(cfg, i, self.pctx) for i in range(cfg.num_hidden_layers)]
        else:
            self.layers = [DecoderLayer(cfg, i, self.pctx, ep_mode) for i in range(cfg.num_hidden_layers)]
        self.embed: Optional[torch.Tensor] = None
        self.final_norm: Optional[torch.Tensor] = None
        self.lm_head: Optional[LinearWeight] = None          # vocab-parallel slice under TP
        self.rope_cache: Optional[torch.Tensor] = None
        self.mtp = None
        if (with_mtp if with_mtp is not None else cfg.mtp_num_layers > 0):
            from .mtp import MTPHead
            self.mtp = MTPHead(cfg, self.pctx, ep_mode)
        tp = self.pctx.tp_size
        self.vocab_parallel = tp > 1 and cfg.vocab_size % tp == 0
        self.sp_capacity_hint = 0            # the engine sets this to its largest step so the area is allocated once
        # layers whose output (the residual stream after the layer) is kept per step for a conditioned draft model
        self.capture_layers: Tuple[int, ...] = ()
        self.aux_hidden: List[torch.Tensor] = []
        self.dflash = None                   # models.dflash.BlockDiffusionDrafter
        self.vision = None                   # models.vision.VisionTower (multimodal checkpoints)

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02, max_pos: Optional[int] = None) -> "DecoderLM":
        cfg, dev, dt = self.cfg, self.device, self.dtype
        gen_dev = "cuda" if dev.type == "cuda" else "cpu"
        gen = torch.Generator(device=gen_dev)
        gen.manual_seed(seed)
        self.embed = randn_weight(gen, cfg.vocab_size, cfg.hidden_size, std, dt, dev)
        for layer in self.layers:
            layer.init_random(gen, std, dt, dev)
        base = 0.0 if cfg.norm_plus_one else 1.0
        self.final_norm = torch.full((cfg.hidden_size,), base, dtype=dt, device=dev)
        head = self.embed if cfg.tie_word_embeddings else randn_weight(gen, cfg.vocab_size, cfg.hidden_size, std, dt, dev)
        self.set_lm_head(head)
        if self.mtp is not None:
            self.mtp.init_random(gen, std, dt, dev)
        self.finalize(max_pos)
        return self

    def enable_lora(self, max_slots: int = 7):
        """Attach one adapter set to the attention, dense-FFN and mixture-of-experts blocks of every layer."""
        from ..lora import LoraSet
        if getattr(self, "lora", None) is None:
            self.lora = LoraSet(max_slots)
            for l in self.layers:
                if l.kind == "attention":
                    l.mixer.lora = self.lora
                l.ffn.lora, l.ffn.lora_prefix = self.lora, f"layers.{l.idx}.mlp."
                shared = getattr(l.ffn, "shared", None)
                if shared is not None:
                    shared.lora, shared.lora_prefix = self.lora, f"layers.{l.idx}.mlp.shared_expert."
        return self.lora

    def set_kv_rotation(self, on: bool = True) -> bool:
        """"turbo8" cache: every plain attention layer (the draft head's included) rotates its q / k / v heads with the
        orthonormal Walsh-Hadamard transform before the FP8 cache write and rotates the attention output back.  Dot
        products are unchanged (the transform is orthogonal), rotated coordinates are near-Gaussian, so the FP8 range
        is not spent on a few outlier channels.  Returns False (nothing changed) when the model has layers the rotation
        does not cover: latent attention, or a head size other than 128 with full rotary width on the GPU.
        Reference: ``kernels/gb10/common/reshape_and_cache_turbo.cu`` (turbo8 = WHT + e4m3)."""
        from ..layers.attention import Attention
        cfg = self.cfg
        d = cfg.head_dim
        if cfg.kv_lora_rank > 0 or d & (d - 1):
            return False
        if self.device.type == "cuda" and not (d == 128 and cfg.rotary_dim == 128):
            return False
        layers = list(self.layers) + ([self.mtp.layer] if self.mtp is not None else [])
        for l in layers:
            if isinstance(getattr(l, "mixer", None), Attention):
                l.mixer.kv_rotate = bool(on)
        return True

    def register_adapter(self, adapter) -> int:
        """Make ``adapter`` (whole, as loaded) resident on this rank, cut like the base weights; returns its slot."""
        from ..lora import localize
        return self.enable_lora().register(localize(adapter, self))

    def set_lm_head(self, head: torch.Tensor) -> None:
        if self.vocab_parallel:
            head = shard_rows(head, self.pctx.tp_rank, self.pctx.tp_size).contiguous()
        self.lm_head = LinearWeight("dense", head)

    def finalize(self, max_pos: Optional[int] = None) -> None:
        cfg = self.cfg
        mp = max_pos or cfg.max_position_embeddings
        self.rope_cache = ref.build_rope_cache(cfg.rotary_dim, mp, cfg.rope_theta, cfg.rope_scaling, self.device)
        if cfg.rope_local_theta:
            local = ref.build_rope_cache(cfg.rotary_dim, mp, cfg.rope_local_theta, None, self.device)
            for l in self.layers:
                if l.kind == "attention" and getattr(l.mixer, "local", False):
                    l.rope_override = local

    # ------------------------------------------------------------------ cache allocation
    def attention_layers(self) -> List[int]:
        return [l.idx for l in self.layers if l.kind == "attention"]

    def gdn_layers(self) -> List[int]:
        """Layers with a recurrent state slot (Gated DeltaNet or Mamba-2)."""
        return [l.idx for l in self.layers if l.kind in ("gdn", "mamba2")]

    def kv_bytes_per_block(self, block_size: int, kv_dtype: torch.dtype, high_precision_layers=()) -> int:
        n_attn = len(self.attention_layers()) + (1 if self.mtp is not None else 0)
        hkv = self.layers[self.attention_layers()[0]].mixer.hkv if n_attn else 0
        n_hi = len([i for i in self.attention_layers() if i in set(high_precision_layers)])
        per = 2 * block_size * hkv * self.cfg.head_dim
        return int(per * ((n_attn - n_hi) * kv_element_bytes(kv_dtype) + n_hi * max(2.0, kv_element_bytes(kv_dtype))))

    def alloc_cache(self, num_blocks: int, block_size: int, kv_dtype: torch.dtype, state_slots: int = 0,
                    high_precision_layers=()) -> CacheStore:
        """``high_precision_layers``: attention layers whose cache stays in 16 bits when ``kv_dtype`` is FP8 or NVFP4 (the
        layers most sensitive to KV quantisation, typically the first and last ones)."""
        store = CacheStore(block_size=block_size, num_blocks=num_blocks)
        hi = set(high_precision_layers)
        for l in self.layers:
            if l.kind == "attention":
                dt = (torch.bfloat16 if self.dtype == torch.bfloat16 else self.dtype) if (l.idx in hi and kv_dtype_is_quantised(kv_dtype)) else kv_dtype
                store.kv[l.idx] = alloc_kv(num_blocks, block_size, l.mixer.hkv, self.cfg.head_dim, dt, self.device)
                store.kv_scales[l.idx] = (1.0, 1.0)
            elif l.kind in ("gdn", "mamba2"):
                store.states[l.idx] = l.mixer.alloc_state(max(1, state_slots), self.device, self.dtype)
        if self.mtp is not None:
            self.mtp.alloc_cache(store, num_blocks, block_size, kv_dtype, self.device)
        return store

    # ------------------------------------------------------------------ forward
    def embed_tokens(self, ids: torch.Tensor) -> torch.Tensor:
        from ..ops import checked
        if checked.ENABLED:
            checked.index_range("input_ids", ids, 0, self.cfg.vocab_size)
        e = self.embed[ids.long()]
        if self.cfg.embed_scale != 1.0:
            e = e * torch.tensor(self.cfg.embed_scale, dtype=e.dtype)      # the factor is rounded to the weight dtype first
        return e

    # ------------------------------------------------------------------ sequence-parallel prefill (tensor parallel)
    def _seq_parallel_area(self, batch: ForwardBatch, T: int):
        """The peer-memory area for a sequence-parallel step, or None when this step takes the replicated path.
        Decided from the model, the configuration and the step's row count only, so every rank decides alike."""
        p = self.pctx
        if p.tp_size <= 1 or p.comm is None or not hasattr(p.comm, "seq_parallel"):
            return None
        # prefill-size steps are owned in 128-row blocks; pure decode steps of at most 128 rows are owned row by row
        # (every rank reduces and normalises T / world rows), which pays off once the all-reduce latency of a wide
        # group dominates the step
        decode_sp = (SEQ_PARALLEL_DECODE_MIN_WORLD > 0 and p.tp_size >= SEQ_PARALLEL_DECODE_MIN_WORLD and T <= 128
                     and batch.num_decodes == batch.num_seqs and batch.max_query_len == 1)
        if T < SEQ_PARALLEL_MIN_TOKENS and not decode_sp:
            return None
        if batch.adapter_rows is not None or self.device.type != "cuda" or ops.FORCE_REFERENCE:
            return None
        if torch.cuda.is_current_stream_capturing():
            # a captured step may use an area that already exists (the eager passes before the capture create it); it
            # must never allocate or rendezvous
            areas = getattr(p.comm, "_sp_areas", None)
            area = areas.get(self.cfg.hidden_size) if (decode_sp and areas) else None
            if area is None or area.t_pad < T or not getattr(self, "_sp_model_ok", False):
                return None
            return area
        ok = getattr(self, "_sp_model_ok", None)
        if ok is None:
            ok = self.dtype == torch.bfloat16 and self.cfg.hidden_size % 256 == 0 and not self.cfg.sandwich_norms and all(
                l.kind == "attention" and not l.is_moe and l.ffn.shard and l.mixer.qkv.kind == "fp8_block"
                and l.mixer.o.kind == "fp8_block" and l.ffn.gate_up.kind == "fp8_block" and l.ffn.down.kind == "fp8_block"
                and l.mixer.o.bias is None and l.ffn.down.bias is None for l in self.layers)
            self._sp_model_ok = ok
        if not ok:
            return None
        return p.comm.seq_parallel(max(T, self.sp_capacity_hint), self.cfg.hidden_size)

    def _forward_seq_parallel(self, x: torch.Tensor, batch: ForwardBatch, cache: CacheStore, sp) -> torch.Tensor:
        """Dense tensor-parallel layers with a row-sharded residual stream: every row-parallel GEMM scatters its
        partial tiles to the row owners, the owner reduces, normalises and quantises its rows once and gathers them to
        all ranks, and the next column-parallel GEMM consumes the rows as they arrive."""
        cfg = self.cfg
        eps, p1 = cfg.rms_norm_eps, cfg.norm_plus_one
        res = sp.residual_shard(x)
        act, _ = ops.rmsnorm_act(x, self.layers[0].input_norm, eps, None, p1, True)
        n = len(self.layers)
        hidden = None
        for i, layer in enumerate(self.layers):
            out = layer.mixer.mix(act, batch, cache.layer_kv(layer.idx), self.rope_cache)
            sp.gemm_rs(out if isinstance(out, Act) else Act(x=out), layer.mixer.o)
            act = sp.reduce_norm(res, layer.post_norm, eps, p1)
            sp.gemm_rs(layer.ffn.hidden_act(act), layer.ffn.down)
            if i + 1 < n:
                act = sp.reduce_norm(res, self.layers[i + 1].input_norm, eps, p1)
            else:
                hidden = sp.reduce_hidden(res)
        self.last_prenorm = (hidden, None)
        y, _ = ops.rmsnorm(hidden, self.final_norm, eps, None, p1)
        return y

    @torch.inference_mode()
    def forward(self, batch: ForwardBatch, cache: CacheStore, layer_ids: Optional[List[int]] = None) -> torch.Tensor:
        """Returns the final-normed hidden states ``[T,H]`` of every row.  ``layer_ids`` runs only those layers, in
        order (the layer-skipping draft pass of self-speculative decoding: the kept layers read and write their own KV
        entries, the skipped ones are not touched)."""
        x = batch.inputs_embeds if batch.inputs_embeds is not None else self.embed_tokens(batch.input_ids)
        sp = self._seq_parallel_area(batch, x.shape[0]) if (not self.capture_layers and layer_ids is None) else None
        if sp is not None:
            return self._forward_seq_parallel(x, batch, cache, sp)
        residual = None
        if batch.inputs_embeds is not None:
            x = x.clone()                     # fused epilogues update the residual stream in place
        if layer_ids is not None:
            layers = [self.layers[i] for i in layer_ids]
            for k, layer in enumerate(layers):
                nxt = layers[k + 1] if k + 1 < len(layers) else None
                next_norm = nxt.input_norm if (nxt is not None and nxt.accepts_prenormed()) else None
                x, residual = layer.forward(x, residual, batch, cache, self.rope_cache, next_norm=next_norm)
            y, _ = ops.rmsnorm(x, self.final_norm, self.cfg.rms_norm_eps, residual, self.cfg.norm_plus_one)
            return y
        n = len(self.layers)
        self.aux_hidden = []
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1] if i + 1 < n else None
            next_norm = nxt.input_norm if (nxt is not None and nxt.accepts_prenormed()) else None
            x, residual = layer.forward(x, residual, batch, cache, self.rope_cache, next_norm=next_norm)
            if i in self.capture_layers:
                # the stream after layer i: already summed when the layer's epilogue handed over normalised activations
                self.aux_hidden.append(residual.clone() if isinstance(x, Act) else (x + residual if residual is not None else x.clone()))
        self.last_prenorm = (x, residual)
        y, _ = ops.rmsnorm(x, self.final_norm, self.cfg.rms_norm_eps, residual, self.cfg.norm_plus_one)
        return y

    @torch.inference_mode()
    def compute_logits(self, hidden: torch.Tensor, indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        h = hidden if indices is None else hidden[indices]
        logits = ops.linear(h, self.lm_head)
        if self.vocab_parallel and self.pctx.comm is not None:
            logits = self.pctx.comm.all_gather(logits, dim=-1)
        cap = self.cfg.final_logit_softcapping
        if cap:
            logits = torch.tanh(logits.float() / cap).mul_(cap).to(logits.dtype)
        return logits

    def build_draft_head(self, row_ids: List[int], kind: str = "fp8_block") -> None:
        """A draft-only language-model head over the token ids ``row_ids`` (ascending), quantised to ``kind``: draft
        steps score these rows instead of the whole vocabulary (``draft_top1``).  On a vocabulary-parallel rank the head
        holds the chosen rows of this rank's shard.  Reference: ``crates/spark-model/src/layers/mtp_head/ranked_head.rs``
        (draft-only quantised head built from ranked rows of the full head)."""
        ids = torch.tensor(sorted(int(t) for t in row_ids), dtype=torch.long)
        lo = 0
        if self.vocab_parallel:
            shard = self.cfg.vocab_size // self.pctx.tp_size
            lo = self.pctx.tp_rank * shard
            ids = ids[(ids >= lo) & (ids < lo + shard)]
        if ids.numel() == 0:
            ids = torch.tensor([lo], dtype=torch.long)          # a rank never holds an empty head
        n = int(ids.numel())
        if self.device.type == "cuda" and n % 128:
            # the GEMM tiles want a multiple of 128 rows: repeat the last row (same logit, same token id, so the
            # argmax is unchanged) rather than add zero rows that could win against negative logits
            ids = torch.cat([ids, ids[-1:].expand(128 - n % 128)])
        w = self.lm_head.dequantized()[(ids - lo).to(self.lm_head.weight.device)]
        if kind == "fp8_block" and (w.shape[1] % 128 or not w.is_floating_point()):
            kind = "dense"
        self.draft_head = LinearWeight.from_dense(w.contiguous(), kind)
        self.draft_row_ids = ids.to(self.device)
        self.draft_rows = n

    @torch.inference_mode()
    def draft_top1(self, hidden: torch.Tensor, want_logprob: bool = False):
        """``(token ids [B], ln p(top-1) [B] or None)`` of a draft step: over the draft head's rows when one was built,
        over the whole vocabulary otherwise.  The probability is taken over the rows that were scored."""
        if getattr(self, "draft_head", None) is None:
            lg = self.compute_logits(hidden)
            tok = ops.argmax(lg)
            lp = lg.float().log_softmax(-1).gather(-1, tok.view(-1, 1).long())[:, 0] if want_logprob else None
            return tok, lp
        lg = ops.linear(hidden, self.draft_head)
        cap = self.cfg.final_logit_softcapping
        if cap:
            lg = torch.tanh(lg.float() / cap).mul_(cap).to(lg.dtype)
        idx, val = ops.argmax(lg, with_value=True)
        tok = self.draft_row_ids[idx.long()]
        lse = torch.logsumexp(lg[:, :self.draft_rows].float(), -1) if want_logprob else None      # not the repeated rows
        if self.vocab_parallel and self.pctx.comm is not None:
            cols = [val.double(), tok.double()] + ([lse.double()] if want_logprob else [])
            allp = self.pctx.comm.all_gather(torch.stack(cols, 1), dim=1).view(val.shape[0], self.pctx.tp_size, len(cols))
            best = ref.argmax_first(allp[..., 0])
            tok = allp[..., 1].gather(1, best[:, None])[:, 0].to(torch.int64)
            val = allp[..., 0].gather(1, best[:, None])[:, 0]
            if want_logprob:
                lse = torch.logsumexp(allp[..., 2], -1)
        lp = (val.float() - lse.float()) if want_logprob else None
        return tok, lp

    @torch.inference_mode()
    def greedy_tokens(self, hidden: torch.Tensor, indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Argmax token per row without materialising the full-vocabulary logits on any rank: each rank takes the
        argmax of its vocabulary shard, the ranks exchange one (max, index) pair per row and the best shard wins
        (ties go to the lowest global index).  Replaces the all-gather of ``[rows, vocab]`` logits of
        :meth:`compute_logits` when every row of the step is plain greedy."""
        h = hidden if indices is None else hidden[indices]
        logits = ops.linear(h, self.lm_head)
        idx, val = ops.argmax(logits, with_value=True)
        if not (self.vocab_parallel and self.pctx.comm is not None):
            return idx
        shard = self.cfg.vocab_size // self.pctx.tp_size
        pair = torch.stack([val.double(), (idx + self.pctx.tp_rank * shard).double()], dim=1)       # [B, 2], exact
        allp = self.pctx.comm.all_gather(pair, dim=1).view(pair.shape[0], self.pctx.tp_size, 2)
        vals, ids = allp[..., 0], allp[..., 1]
        best = ref.argmax_first(vals)
        return ids.gather(1, best[:, None])[:, 0].to(torch.int64)

    def commit_spec(self, accepted_rows: List[int], cache: CacheStore) -> None:
        """After speculative verification: fold the accepted rows into every GDN layer's state."""
        for l in self.layers:
            if l.kind in ("gdn", "mamba2"):
                l.mixer.commit(accepted_rows, cache.states[l.idx])

    # ------------------------------------------------------------------ oracle
    @torch.inference_mode()
    def forward_dense_reference(self, token_ids: List[int]) -> torch.Tensor:
        """Plain eager forward of ONE sequence without any paging (logits of every position).

        Used by tests as the "plain eager forward" that the paged/batched engine must match.
        """
        n = len(token_ids)
        bs = 16
        nblk = (n + bs - 1) // bs
        kv_dtype = self.dtype
        tmp = self.alloc_cache(nblk, bs, kv_dtype, state_slots=1)
        fb = ForwardBatch.build([list(token_ids)], [0], [list(range(nblk))], bs, device=self.device,
                                state_slots=[0], has_state=[False], all_logits=True)
        h = self.forward(fb, tmp)
        return self.compute_logits(h)
