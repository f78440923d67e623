"""Model / quantization / serving configuration.

`ModelConfig.from_hf` parses a HuggingFace ``config.json`` dictionary into one
flat dataclass that every layer reads.  It covers the decoder families the
engine serves: Llama/Mistral/Qwen2/Qwen3 dense, Qwen3-MoE, and the Qwen3-Next
hybrid (Gated-DeltaNet + gated attention + MoE + MTP head).

Reference parity: ``crates/avarok-core/src/config.rs`` (``ModelConfig::from_hf``),
``crates/avarok-core/src/config/dispatch.rs`` (model_type aliases) and
``crates/avarok-core/src/config/methods.rs:187`` (``local_expert_range``).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

# model_type spellings accepted from config.json -> canonical family.
_FAMILY_ALIASES = {
    "llama": "dense", "mistral": "dense", "qwen2": "dense", "qwen3": "dense", "gemma3_text": "dense", "gemma3": "dense",
    "qwen3_moe": "moe", "qwen3_vl_moe": "moe", "mixtral": "moe", "minimax_m2": "moe",
    "qwen3_next": "hybrid", "qwen3_5": "hybrid", "qwen35": "hybrid", "qwen3_5_text": "hybrid",
    "qwen3_5_moe": "hybrid", "qwen35_moe": "hybrid", "qwen3_6_moe": "hybrid", "qwen3_5_moe_text": "hybrid",
    "holo3_1_moe": "hybrid",
    "nemotron_h": "hybrid", "nemotron_h_puzzle": "hybrid",
    "deepseek_v2": "moe", "deepseek_v3": "moe", "deepseek_v32": "moe", "kimi_k2": "moe",
}


@dataclass
class QuantConfig:
    """Weight / KV-cache quantization description.

    method:
      * ``"none"``      – weights stay in ``ModelConfig.dtype``.
      * ``"fp8_block"`` – FP8 e4m3 weights with one fp32 scale per 128x128 tile
        (``weight_scale_inv`` tensors), activations quantized per token per
        128-wide K group at run time.
      * ``"nvfp4"``     – packed E2M1 weights ``[N, K/2]``, e4m3 scale per 16
        elements ``[N, K/16]`` and one fp32 global scale ``weight_scale_2``.
    Reference parity: ``crates/spark-model/src/quant_format/{fp8_blockscaled,modelopt,compressed_tensors}.rs``.
    """
    method: str = "none"
    weight_block: Tuple[int, int] = (128, 128)
    group_size: int = 16
    kv_cache_dtype: str = "auto"  # auto | bf16 | fp8 | turbo8 (Hadamard-rotated fp8) | nvfp4
    # modules kept in high precision (substring match on parameter prefix)
    ignore: List[str] = field(default_factory=lambda: ["lm_head", "embed_tokens", "router", "gate."])
    # when method is nvfp4 for experts only (config 3: attention bf16, experts nvfp4)
    experts_only: bool = False

    @staticmethod
    def from_hf(qc: Optional[Dict[str, Any]]) -> "QuantConfig":
        if not qc:
            return QuantConfig()
        method = str(qc.get("quant_method", qc.get("quant_algo", ""))).lower()
        fmt = str(qc.get("fmt", qc.get("format", ""))).lower()
        if method == "fp8" or "fp8" in method:
            wb = qc.get("weight_block_size") or [128, 128]
            return QuantConfig(method="fp8_block", weight_block=(int(wb[0]), int(wb[1])),
                               kv_cache_dtype="fp8" if qc.get("kv_cache_scheme") else "auto")
        if "nvfp4" in method or "nvfp4" in fmt or method in ("modelopt", "modelopt_fp4"):
            gs = int(qc.get("group_size", 16))
            ign = list(qc.get("ignore", qc.get("exclude_modules", [])))
            out = QuantConfig(method="nvfp4", group_size=gs)
            if ign:
                out.ignore = ign
            return out
        if method == "compressed-tensors":
            groups = qc.get("config_groups", {})
            for g in groups.values():
                w = g.get("weights", {})
                if w.get("num_bits") == 4 and w.get("type") == "float":
                    return QuantConfig(method="nvfp4", group_size=int(w.get("group_size", 16)),
                                       ignore=list(qc.get("ignore", [])) or QuantConfig().ignore)
                if w.get("num_bits") == 8 and w.get("type") == "float":
                    return QuantConfig(method="fp8_block")
        return QuantConfig()


@dataclass
class ModelConfig:
    model_type: str = "llama"
    family: str = "dense"            # dense | moe | hybrid
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    partial_rotary_factor: float = 1.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = False             # Qwen3-style per-head RMSNorm on q and k
    attn_output_gate: bool = False    # Qwen3-Next gated attention (q_proj emits q and gate)
    sliding_window: Optional[int] = None
    norm_plus_one: bool = False       # (1 + weight) RMSNorm convention (Qwen3-Next, Gemma)
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_scoring: str = "softmax"   # softmax | sigmoid | sqrtsoftplus
    routed_scaling_factor: float = 1.0
    router_n_group: int = 0           # group-limited routing (DeepSeek-V3): experts split into n_group groups ...
    router_topk_group: int = 0        # ... of which the topk_group best stay eligible
    router_selection_bias: bool = False   # per-expert e_score_correction_bias used for selection only
    num_hash_layers: int = 0          # first MoE layers select experts by a static token-id table (DeepSeek-V4)
    decoder_sparse_step: int = 1
    mlp_only_layers: List[int] = field(default_factory=list)
    # hybrid (Gated DeltaNet)
    layer_types: List[str] = field(default_factory=list)  # "full_attention" | "linear_attention"
    full_attention_interval: int = 4
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    # single-module blocks (Nemotron-H): per layer "mamba" | "attention" | "mlp"; empty for the other families
    block_types: List[str] = field(default_factory=list)
    mamba_num_heads: int = 0
    mamba_head_dim: int = 64
    ssm_state_size: int = 128
    mamba_n_groups: int = 8
    mamba_conv_kernel: int = 4
    mamba_dt_min: float = 0.0
    mlp_activation: str = "silu_glu"  # silu_glu (gated SwiGLU) | relu2 (up -> relu^2 -> down)
    # multi-head latent attention (DeepSeek): 0 = plain GQA.  head_dim is then the padded cache width
    kv_lora_rank: int = 0
    q_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    rope_interleaved: bool = True     # checkpoint stores rotary columns as (even, odd) pairs
    first_k_dense_replace: int = 0    # leading layers with a dense FFN in an otherwise MoE model
    # Gemma: scaled embeddings, explicit attention scale, norms after the mixer and the FFN as well as before them, a
    # separate rotary base for sliding-window layers, soft-capped output logits
    embed_scale: float = 1.0
    attn_scale: float = 0.0           # 0 = head_dim ** -0.5
    sandwich_norms: bool = False
    rope_local_theta: float = 0.0     # rotary base of the sliding-window layers (0 = same table as the other layers)
    final_logit_softcapping: float = 0.0
    # multimodal: interleaved MRoPE sections (time, row, column), the image placeholder id and the vision tower's config
    mrope_section: List[int] = field(default_factory=list)
    image_token_id: int = -1
    vision: Any = None                # models.vision.VisionConfig
    # MTP speculative head
    mtp_num_layers: int = 0
    # numerics
    dtype: str = "bfloat16"
    quant: QuantConfig = field(default_factory=QuantConfig)
    bos_token_id: Optional[int] = None
    eos_token_id: Any = None

    # ------------------------------------------------------------------ helpers
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    def layer_kind(self, i: int) -> str:
        """Mixer kind of layer ``i``: ``attention``, ``gdn``, ``mamba2`` or ``none`` (an FFN-only block)."""
        if self.block_types:
            return {"mamba": "mamba2", "attention": "attention"}.get(self.block_types[i], "none")
        if self.family != "hybrid":
            return "attention"                # (Gemma's layer_types only choose the attention window)
        if self.layer_types:
            return "attention" if self.layer_types[i] == "full_attention" else "gdn"
        return "attention" if (i + 1) % self.full_attention_interval == 0 else "gdn"

    def is_moe_layer(self, i: int) -> bool:
        if self.block_types:
            return self.block_types[i] == "moe"
        if self.num_experts <= 0 or i in self.mlp_only_layers or i < self.first_k_dense_replace:
            return False
        return (i + 1) % max(1, self.decoder_sparse_step) == 0

    def local_expert_range(self, ep_rank: int, ep_size: int) -> Tuple[int, int]:
        """Contiguous expert slice owned by ``ep_rank`` (remainder to the low ranks)."""
        e = self.num_experts
        base, rem = divmod(e, ep_size)
        lo = ep_rank * base + min(ep_rank, rem)
        return lo, lo + base + (1 if ep_rank < rem else 0)

    def eos_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, (list, tuple)):
            return [int(x) for x in self.eos_token_id]
        return [int(self.eos_token_id)]

    def param_count(self) -> int:
        h, L = self.hidden_size, self.num_hidden_layers
        n = self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        for i in range(L):
            if self.layer_kind(i) == "attention":
                qmul = 2 if self.attn_output_gate else 1
                n += h * (self.q_size * qmul + 2 * self.kv_size) + self.q_size * h
            elif self.layer_kind(i) == "mamba2":
                di = self.mamba_num_heads * self.mamba_head_dim
                n += h * (2 * di + 2 * self.mamba_n_groups * self.ssm_state_size + self.mamba_num_heads) + di * h
            elif self.layer_kind(i) == "none":
                pass
            else:
                kd = self.linear_num_key_heads * self.linear_key_head_dim
                vd = self.linear_num_value_heads * self.linear_value_head_dim
                n += h * (2 * kd + 2 * vd) + h * 2 * self.linear_num_value_heads + vd * h
            if self.is_moe_layer(i):
                n += self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
                n += 3 * h * self.shared_expert_intermediate_size
            elif self.block_types:
                n += 2 * h * self.intermediate_size if self.block_types[i] == "mlp" else 0
            else:
                n += 3 * h * self.intermediate_size
        return n

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_hf(cfg: Dict[str, Any]) -> "ModelConfig":
        outer = cfg
        if "text_config" in cfg and isinstance(cfg["text_config"], dict):
            merged = dict(cfg["text_config"])
            for k in ("quantization_config", "torch_dtype"):
                if k in cfg and k not in merged:
                    merged[k] = cfg[k]
            cfg = merged
        mt = str(cfg.get("model_type", "llama")).lower()
        if mt not in _FAMILY_ALIASES:
            raise ValueError(f"Unsupported model_type '{mt}'. Supported: {sorted(_FAMILY_ALIASES)}")
        fam = _FAMILY_ALIASES[mt]
        nh = int(cfg["num_attention_heads"])
        hs = int(cfg["hidden_size"])
        rope_params = cfg.get("rope_parameters") or {}
        c = ModelConfig(
            model_type=mt, family=fam,
            vocab_size=int(cfg["vocab_size"]), hidden_size=hs,
            intermediate_size=int(cfg.get("intermediate_size", 0) or 0),
            num_hidden_layers=int(cfg.get("num_hidden_layers") or len(cfg.get("layers_block_type") or cfg.get("hybrid_override_pattern") or [])),
            num_attention_heads=nh,
            num_key_value_heads=int(cfg.get("num_key_value_heads", nh)),
            head_dim=int(cfg.get("head_dim") or hs // nh),
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
            rope_theta=float(cfg.get("rope_theta", rope_params.get("rope_theta", 10000.0))),
            rope_scaling=cfg.get("rope_scaling") or (rope_params if rope_params.get("rope_type", "default") != "default" else None),
            partial_rotary_factor=float(cfg.get("partial_rotary_factor", rope_params.get("partial_rotary_factor", 1.0))),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 32768)),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            attention_bias=bool(cfg.get("attention_bias", mt == "qwen2")),
            qk_norm=mt in ("qwen3", "qwen3_moe", "qwen3_vl_moe") or fam == "hybrid",
            attn_output_gate=fam == "hybrid" and bool(cfg.get("attn_output_gate", True)),
            sliding_window=cfg.get("sliding_window") if cfg.get("use_sliding_window", True) else None,
            norm_plus_one=fam == "hybrid",
            num_experts=int(cfg.get("num_experts", cfg.get("num_local_experts", 0)) or 0),
            num_experts_per_tok=int(cfg.get("num_experts_per_tok", 0) or 0),
            moe_intermediate_size=int(cfg.get("moe_intermediate_size", 0) or 0),
            shared_expert_intermediate_size=int(cfg.get("shared_expert_intermediate_size", 0) or 0),
            norm_topk_prob=bool(cfg.get("norm_topk_prob", True)),
            router_scoring=str(cfg.get("scoring_func", "softmax")),
            routed_scaling_factor=float(cfg.get("routed_scaling_factor", 1.0) or 1.0),
            router_n_group=int(cfg.get("n_group", 0) or 0),
            router_topk_group=int(cfg.get("topk_group", 0) or 0),
            router_selection_bias=bool(cfg.get("router_selection_bias", cfg.get("topk_method", "") == "noaux_tc")),
            num_hash_layers=int(cfg.get("num_hash_layers", 0) or 0),
            decoder_sparse_step=int(cfg.get("decoder_sparse_step", 1) or 1),
            mlp_only_layers=list(cfg.get("mlp_only_layers", []) or []),
            layer_types=list(cfg.get("layer_types", []) or []),
            full_attention_interval=int(cfg.get("full_attention_interval", 4) or 4),
            linear_num_key_heads=int(cfg.get("linear_num_key_heads", 0) or 0),
            linear_num_value_heads=int(cfg.get("linear_num_value_heads", 0) or 0),
            linear_key_head_dim=int(cfg.get("linear_key_head_dim", 128) or 128),
            linear_value_head_dim=int(cfg.get("linear_value_head_dim", 128) or 128),
            linear_conv_kernel_dim=int(cfg.get("linear_conv_kernel_dim", 4) or 4),
            mtp_num_layers=int(cfg.get("mtp_num_hidden_layers", cfg.get("num_nextn_predict_layers", 0)) or 0),
            dtype=str(cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))),
            quant=QuantConfig.from_hf(cfg.get("quantization_config")),
            bos_token_id=cfg.get("bos_token_id"), eos_token_id=cfg.get("eos_token_id"),
        )
        if mt in ("gemma3_text", "gemma3"):
            rp = cfg.get("rope_parameters") or {}
            glob, loc = rp.get("full_attention") or {}, rp.get("sliding_attention") or {}
            c.rope_theta = float(glob.get("rope_theta", cfg.get("rope_theta", 1e6)))
            c.rope_scaling = glob if glob.get("rope_type", "default") != "default" else cfg.get("rope_scaling")
            c.rope_local_theta = float(loc.get("rope_theta", cfg.get("rope_local_base_freq", 1e4)))
            c.partial_rotary_factor = 1.0
            c.norm_plus_one = c.qk_norm = c.sandwich_norms = True
            c.embed_scale = float(hs) ** 0.5
            c.attn_scale = float(cfg.get("query_pre_attn_scalar", c.head_dim)) ** -0.5
            c.mlp_activation = "gelu_tanh_glu"
            c.layer_types = list(cfg.get("layer_types") or [])
            c.sliding_window = cfg.get("sliding_window")
            c.final_logit_softcapping = float(cfg.get("final_logit_softcapping") or 0.0)
            c.tie_word_embeddings = bool(cfg.get("tie_word_embeddings", True))
            if cfg.get("attn_logit_softcapping"):
                raise ValueError("attention logit soft-capping (Gemma-2) is not supported")
        if mt == "mixtral":
            c.moe_intermediate_size = c.intermediate_size
        if mt.startswith("deepseek") or mt == "kimi_k2":
            c.num_experts = int(cfg.get("n_routed_experts", 0) or 0)
            c.shared_expert_intermediate_size = c.moe_intermediate_size * int(cfg.get("n_shared_experts", 0) or 0)
            c.first_k_dense_replace = int(cfg.get("first_k_dense_replace", 0) or 0)
            c.decoder_sparse_step = int(cfg.get("moe_layer_freq", 1) or 1)
            c.router_scoring = str(cfg.get("scoring_func", "sigmoid" if mt != "deepseek_v2" else "softmax"))
            c.router_selection_bias = mt != "deepseek_v2"
            c.num_key_value_heads = nh
            c.kv_lora_rank = int(cfg.get("kv_lora_rank", 512))
            c.q_lora_rank = int(cfg.get("q_lora_rank") or 0)
            c.qk_nope_head_dim = int(cfg.get("qk_nope_head_dim", 128))
            c.qk_rope_head_dim = int(cfg.get("qk_rope_head_dim", 64))
            c.v_head_dim = int(cfg.get("v_head_dim", 128))
            c.rope_interleaved = bool(cfg.get("rope_interleave", True))
            need = max(c.qk_nope_head_dim + c.qk_rope_head_dim, c.v_head_dim)
            c.head_dim = next((d for d in (64, 128, 256) if d >= need), need)
            c.partial_rotary_factor = c.qk_rope_head_dim / c.head_dim
            c.qk_norm = False
        if mt.startswith("nemotron_h"):
            blocks = cfg.get("layers_block_type")
            if not blocks and cfg.get("hybrid_override_pattern"):
                blocks = [{"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}[ch] for ch in cfg["hybrid_override_pattern"]]
            c.block_types = list(blocks or [])
            c.num_hidden_layers = len(c.block_types)
            c.mamba_num_heads = int(cfg.get("mamba_num_heads", 128))
            c.mamba_head_dim = int(cfg.get("mamba_head_dim", 64))
            c.ssm_state_size = int(cfg.get("ssm_state_size", 128))
            c.mamba_n_groups = int(cfg.get("n_groups", 8))
            c.mamba_conv_kernel = int(cfg.get("conv_kernel", 4))
            c.mamba_dt_min = float(cfg.get("time_step_min", 0.001))
            c.mlp_activation = "relu2"
            c.rms_norm_eps = float(cfg.get("layer_norm_epsilon", cfg.get("rms_norm_eps", 1e-5)))
            c.partial_rotary_factor = 0.0                     # attention blocks carry no positional rotation
            c.qk_norm = c.attn_output_gate = c.norm_plus_one = False
            c.num_experts = c.num_experts_per_tok = 0
            if "moe" in c.block_types:
                raise ValueError("nemotron_h checkpoints with MoE blocks are not supported")
        c.mrope_section = list(rope_params.get("mrope_section") or (cfg.get("rope_scaling") or {}).get("mrope_section") or [])
        if isinstance(outer.get("vision_config"), dict) and outer.get("image_token_id") is not None and fam == "hybrid":
            from .models.vision import VisionConfig
            c.vision = VisionConfig.from_hf(outer["vision_config"])
            c.image_token_id = int(outer["image_token_id"])
            if not c.mrope_section:
                c.mrope_section = [11, 11, 10]
        c.validate()
        return c

    @staticmethod
    def from_pretrained(path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        c = ModelConfig.from_hf(cfg)
        side = os.path.join(path, "hf_quant_config.json")   # ModelOpt sidecar
        if c.quant.method == "none" and os.path.exists(side):
            with open(side) as f:
                q = json.load(f).get("quantization", {})
            c.quant = QuantConfig.from_hf(q)
        return c

    def validate(self) -> None:
        if self.num_attention_heads % max(1, self.num_key_value_heads):
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.num_experts and not self.num_experts_per_tok:
            raise ValueError("MoE config needs num_experts_per_tok")
        if self.family == "hybrid" and not self.linear_num_value_heads and not self.block_types:
            raise ValueError("hybrid config needs linear_num_value_heads")

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


# ---------------------------------------------------------------------------- presets
def tiny_dense(dtype: str = "float32") -> ModelConfig:
    """2-layer plumbing model: hidden 256, 4q/2kv heads x 64, FFN 512, vocab 1024."""
    return ModelConfig(model_type="llama", family="dense", vocab_size=1024, hidden_size=256,
                       intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6,
                       max_position_embeddings=4096, dtype=dtype)


def llama3_8b(quant: str = "fp8_block") -> ModelConfig:
    return ModelConfig(model_type="llama", family="dense", vocab_size=128256, hidden_size=4096,
                       intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                       num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=5e5,
                       max_position_embeddings=8192,
                       quant=QuantConfig(method=quant, kv_cache_dtype="fp8" if quant != "none" else "auto"))


def llama3_70b(quant: str = "fp8_block") -> ModelConfig:
    return ModelConfig(model_type="llama", family="dense", vocab_size=128256, hidden_size=8192,
                       intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                       num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=5e5,
                       max_position_embeddings=65536,
                       quant=QuantConfig(method=quant, kv_cache_dtype="fp8" if quant != "none" else "auto"))


def qwen3_30b_a3b(quant: str = "nvfp4") -> ModelConfig:
    return ModelConfig(model_type="qwen3_moe", family="moe", vocab_size=151936, hidden_size=2048,
                       intermediate_size=6144, num_hidden_layers=48, num_attention_heads=32,
                       num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
                       qk_norm=True, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                       norm_topk_prob=True, max_position_embeddings=40960,
                       quant=QuantConfig(method=quant, experts_only=True, kv_cache_dtype="fp8"))


def qwen3_next_80b(quant: str = "fp8_block") -> ModelConfig:
    return ModelConfig(model_type="qwen3_next", family="hybrid", vocab_size=151936, hidden_size=2048,
                       intermediate_size=5120, num_hidden_layers=48, num_attention_heads=16,
                       num_key_value_heads=2, head_dim=256, rms_norm_eps=1e-6, rope_theta=1e7,
                       partial_rotary_factor=0.25, qk_norm=True, attn_output_gate=True, norm_plus_one=True,
                       num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512,
                       shared_expert_intermediate_size=512, norm_topk_prob=True,
                       full_attention_interval=4, linear_num_key_heads=16, linear_num_value_heads=32,
                       linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4,
                       mtp_num_layers=1, max_position_embeddings=262144,
                       quant=QuantConfig(method=quant, kv_cache_dtype="fp8"))


def tiny_moe(dtype: str = "float32") -> ModelConfig:
    return ModelConfig(model_type="qwen3_moe", family="moe", vocab_size=1024, hidden_size=256,
                       intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, rope_theta=1e6, qk_norm=True,
                       num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                       max_position_embeddings=4096, dtype=dtype)


def tiny_hybrid(dtype: str = "float32") -> ModelConfig:
    return ModelConfig(model_type="qwen3_next", family="hybrid", vocab_size=1024, hidden_size=256,
                       intermediate_size=512, num_hidden_layers=4, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, rope_theta=1e6, partial_rotary_factor=0.25,
                       qk_norm=True, attn_output_gate=True, norm_plus_one=True,
                       num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                       shared_expert_intermediate_size=128, full_attention_interval=4,
                       linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
                       linear_value_head_dim=32, linear_conv_kernel_dim=4, mtp_num_layers=1,
                       max_position_embeddings=4096, dtype=dtype)


def tiny_nemotron_h(dtype: str = "float32") -> ModelConfig:
    """Nemotron-H style stack of single-module blocks: Mamba-2, position-free attention and relu^2 MLP."""
    return ModelConfig(model_type="nemotron_h", family="hybrid", vocab_size=1024, hidden_size=256, intermediate_size=512,
                       num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                       partial_rotary_factor=0.0, rms_norm_eps=1e-5,
                       block_types=["mamba", "mlp", "mamba", "attention", "mlp", "mamba"], mamba_num_heads=8,
                       mamba_head_dim=32, ssm_state_size=32, mamba_n_groups=2, mamba_conv_kernel=4, mamba_dt_min=0.001,
                       mlp_activation="relu2", max_position_embeddings=4096, dtype=dtype)


def tiny_deepseek(dtype: str = "float32") -> ModelConfig:
    """DeepSeek-V3 style: latent attention, a leading dense layer, then MoE layers with a group-limited sigmoid router,
    selection bias, weight scale and an ungated shared expert."""
    return ModelConfig(model_type="deepseek_v3", family="moe", vocab_size=1024, hidden_size=256, intermediate_size=512,
                       num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, head_dim=64,
                       partial_rotary_factor=0.25, kv_lora_rank=64, q_lora_rank=96, qk_nope_head_dim=32, qk_rope_head_dim=16,
                       v_head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                       shared_expert_intermediate_size=128, first_k_dense_replace=1, router_scoring="sigmoid",
                       router_selection_bias=True, router_n_group=4, router_topk_group=2, routed_scaling_factor=2.5,
                       max_position_embeddings=4096, dtype=dtype)


def nemotron_h_8b(quant: str = "none") -> ModelConfig:
    pattern = "M-M-M-MM-M-M-M*-M-M-M*-M-M-M-M*-M-M-M-M*-M-MM-M-M-M-M-M-"
    blocks = [{"M": "mamba", "*": "attention", "-": "mlp"}[ch] for ch in pattern]
    return ModelConfig(model_type="nemotron_h", family="hybrid", vocab_size=131072, hidden_size=4096, intermediate_size=21504,
                       num_hidden_layers=len(blocks), num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       partial_rotary_factor=0.0, rms_norm_eps=1e-5, block_types=blocks, mamba_num_heads=128, mamba_head_dim=64,
                       ssm_state_size=128, mamba_n_groups=8, mamba_conv_kernel=4, mamba_dt_min=0.001, mlp_activation="relu2",
                       max_position_embeddings=8192, quant=QuantConfig(method=quant, kv_cache_dtype="fp8"))


PRESETS = {
    "tiny-dense": tiny_dense, "tiny-moe": tiny_moe, "tiny-hybrid": tiny_hybrid,
    "llama3-8b": llama3_8b, "llama3-70b": llama3_70b,
    "qwen3-30b-a3b": qwen3_30b_a3b, "qwen3-next-80b": qwen3_next_80b,
    "tiny-nemotron-h": tiny_nemotron_h, "nemotron-h-8b": nemotron_h_8b, "tiny-deepseek": tiny_deepseek,
}


@dataclass
class EngineConfig:
    """Serving knobs (same names/defaults as the reference's serve flags,
    ``crates/spark-server/src/cli/serve_args.rs``)."""
    max_seq_len: int = 32768
    block_size: int = 16
    kv_cache_dtype: str = "auto"
    sparse_attention_blocks: int = 0          # > 0: decode attention reads at most this many KV blocks per sequence
    async_decode: bool = True                 # lag-one decode pipeline for plain greedy decode steps (GPU, CUDA graphs)
    kv_high_precision_layers: tuple = ()      # attention layers that keep a 16-bit cache when kv_cache_dtype is fp8
    gpu_memory_utilization: float = 0.90
    num_kv_blocks: Optional[int] = None       # explicit override (tests / CPU)
    max_num_seqs: int = 128
    max_batch_size: int = 128                 # decode batch cap per step
    max_prefill_tokens: int = 8192
    scheduling_policy: str = "fifo"           # fifo | slai
    tbt_deadline_ms: float = 100.0
    enable_prefix_caching: bool = True
    speculative: bool = False
    num_drafts: int = 0
    mtp_gate: bool = True
    mtp_draft_vocab: int = 0                  # > 0: draft steps score this many rows of the lm_head (a quantised draft-only head)
    mtp_vocab_rank: str = "id"                # "id": the first rows; or the path of a ranked-ids table (utils/vocab_rank.py)
    dcut_ratio: float = 0.0                   # > 0: keep this fraction of the batch's draft rows, ranked by drafter confidence
    ngram_speculative: bool = False           # prompt-lookup drafts (no draft model); uses num_drafts
    self_speculative: bool = False            # layer-skipping drafts from the target model itself; uses num_drafts
    self_spec_keep: float = 0.5               # fraction of the layers the draft pass runs (first and last always kept)
    ngram_max: int = 4
    ngram_min: int = 2
    ssm_cache_slots: int = 16
    ssm_checkpoint_interval: int = 256
    swap_space_gb: float = 0.0
    disk_swap_gb: float = 0.0               # file-backed tier below the host tier (0 = off)
    disk_swap_path: str = ""                # directory of the swap file (default: the system temp directory)
    use_cuda_graphs: bool = True
    tp_size: int = 1
    ep_size: int = 1
    seed: int = 0
    admission_watermark_tokens: int = 256     # decode headroom reserved at admission
    request_timeout_s: float = 0.0
