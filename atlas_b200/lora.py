"""PEFT LoRA adapters: loading (``adapter_config.json`` + ``adapter_model.safetensors``) and per-request application
as a batched gather-matrix-vector (shrink then expand) on top of the base projection.

Tensor parallelism: an adapter is cut the way its base projection is (``localize``).  A column-parallel projection
(q / k / v / gate / up) keeps ``A`` whole and this rank's rows of ``B``; a row-parallel one (o / down) keeps ``B`` whole and
this rank's columns of ``A``, so its delta is a partial sum that the layer adds BEFORE the group reduction.

Mixture-of-experts layers: the router (``mlp.gate``) delta is added to the routing logits; rows that carry an adapter
with per-expert matrices (``mlp.experts.<e>.{gate,up,down}_proj``) have their routed-expert output recomputed with the
adapted expert weights (``layers/moe.py::MoE._adapter_rows_forward``).

Reference parity: ``crates/spark-model/src/layers/lora/*`` (adapter pool, bgmv shrink/expand),
``crates/spark-model/src/layers/moe/lora.rs`` (router + routed-expert deltas), ``kernels/gb10/common/lora_bgmv.cu``,
``spark-runtime/src/weights/adapter.rs``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch


@dataclass
class LoraAdapter:
    name: str
    rank: int
    alpha: float
    # module path (e.g. "layers.3.self_attn.q_proj") -> (A [r, in], B [out, r])
    weights: Dict[str, tuple] = field(default_factory=dict)

    @property
    def scaling(self) -> float:
        return self.alpha / max(1, self.rank)

    def expert_layers(self) -> set:
        """Indices of the layers for which this adapter carries per-expert matrices."""
        if getattr(self, "_expert_layers", None) is None:
            self._expert_layers = {int(k.split(".")[1]) for k in self.weights if ".mlp.experts." in k}
        return self._expert_layers


def load_adapter(path: str, model=None) -> LoraAdapter:
    with open(os.path.join(path, "adapter_config.json")) as f:
        cfg = json.load(f)
    from safetensors.torch import load_file
    st = load_file(os.path.join(path, "adapter_model.safetensors"))
    ad = LoraAdapter(os.path.basename(path.rstrip("/")), int(cfg.get("r", 8)), float(cfg.get("lora_alpha", 16)))
    a_parts, b_parts = {}, {}
    for k, v in st.items():
        key = k.replace("base_model.model.", "").replace("model.", "", 1)
        if ".lora_A" in key:
            a_parts[key.split(".lora_A")[0]] = v
        elif ".lora_B" in key:
            b_parts[key.split(".lora_B")[0]] = v
    dev = model.device if model is not None else "cpu"
    for mod, a in a_parts.items():
        if mod in b_parts:
            ad.weights[mod] = (a.to(dev), b_parts[mod].to(dev))
    return ad


GATE_SUFFIX = "#gate"      # the output-gate half of a gated q_proj (rows [q | gate] per head in the checkpoint)


def localize(adapter: LoraAdapter, model) -> LoraAdapter:
    """This rank's view of ``adapter`` for ``model``: every pair cut like the base projection it updates.  With a
    tensor parallel size of 1 only the gated q_proj split applies."""
    from .layers.attention import Attention
    from .layers.common import shard_cols, shard_rows
    tp, r = model.pctx.tp_size, model.pctx.tp_rank
    out = LoraAdapter(adapter.name, adapter.rank, adapter.alpha)
    for mod, (A, B) in adapter.weights.items():
        parts = mod.split(".")
        known = len(parts) >= 4 and parts[0] == "layers" and parts[1].isdigit() and int(parts[1]) < len(model.layers)
        if known:
            layer, leaf = model.layers[int(parts[1])], parts[-1]
            if parts[2] == "self_attn" and isinstance(layer.mixer, Attention):
                at = layer.mixer
                if leaf == "q_proj":
                    if at.gated:
                        Bv = B.view(model.cfg.num_attention_heads, 2, at.d, B.shape[-1])
                        out.weights[mod + GATE_SUFFIX] = (A, shard_rows(Bv[:, 1].reshape(-1, B.shape[-1]), r, tp).contiguous())
                        B = Bv[:, 0].reshape(-1, B.shape[-1])
                    B = shard_rows(B, r, tp)
                elif leaf in ("k_proj", "v_proj"):
                    B = at._kv_slice(B)
                elif leaf == "o_proj":
                    A = shard_cols(A, r, tp)
            elif parts[2] == "mlp" and len(parts) == 4 and not layer.is_moe and getattr(layer.ffn, "shard", False):
                if leaf in ("gate_proj", "up_proj"):
                    B = shard_rows(B, r, tp)
                elif leaf == "down_proj":
                    A = shard_cols(A, r, tp)
        out.weights[mod] = (A.contiguous(), B.contiguous())
    return out


def bgmv(x: torch.Tensor, adapters: Dict[int, tuple], slot_of_row: torch.Tensor, scaling: Dict[int, float]) -> torch.Tensor:
    """Per-row LoRA delta: ``delta[t] = scaling * B_s (A_s x[t])`` with ``s = slot_of_row[t]`` (slot 0 = no adapter)."""
    out = None
    for slot, (A, B) in adapters.items():
        rows = (slot_of_row == slot).nonzero(as_tuple=True)[0]
        if rows.numel() == 0:
            continue
        d = (x[rows].float() @ A.float().t()) @ B.float().t() * scaling[slot]
        if out is None:
            out = torch.zeros(x.shape[0], B.shape[0], dtype=torch.float32, device=x.device)
        out.index_add_(0, rows, d)
    return out


class LoraSet:
    """Adapters resident on the device, addressed by slot (0 = base model).  ``delta(module, x, rows)`` gives the
    low-rank update of one projection for a batch whose rows may belong to different adapters (or none).

    Supported targets: the dense projections of attention and the SwiGLU FFN (``q/k/v/o_proj``, ``gate/up/down_proj``),
    the shared expert, the router and the routed experts of a mixture-of-experts layer.  Adapters are registered in the
    form ``localize`` gives them, so the set works on a tensor-parallel rank as it does on a whole model."""

    def __init__(self, max_slots: int = 7):       # the device kernel takes slots 1..7
        self.max_slots = max_slots
        self.slots: Dict[int, LoraAdapter] = {}
        self.by_name: Dict[str, int] = {}

    def register(self, adapter: LoraAdapter) -> int:
        if adapter.name in self.by_name:
            slot = self.by_name[adapter.name]
        else:
            free = [s for s in range(1, self.max_slots + 1) if s not in self.slots]
            if not free:
                raise RuntimeError(f"all {self.max_slots} adapter slots are in use")
            slot = free[0]
        self.slots[slot], self.by_name[adapter.name] = adapter, slot
        return slot

    def unregister(self, name: str) -> None:
        slot = self.by_name.pop(name, None)
        if slot is not None:
            self.slots.pop(slot, None)

    def slot_of(self, name: Optional[str]) -> int:
        return self.by_name.get(name, 0) if name else 0

    def delta(self, module: str, x: torch.Tensor, slot_of_row: torch.Tensor) -> Optional[torch.Tensor]:
        ads, sc = {}, {}
        for slot, ad in self.slots.items():
            w = ad.weights.get(module)
            if w is not None:
                ads[slot], sc[slot] = w, ad.scaling
        if not ads:
            return None
        return bgmv(x, ads, slot_of_row, sc)


def add_delta(y: torch.Tensor, lora: Optional["LoraSet"], module: str, x: torch.Tensor, batch, col0: int = 0,
              cols: Optional[int] = None) -> None:
    """``y[:, col0:col0+cols] += delta`` in place when the batch carries adapter rows and an adapter targets ``module``."""
    rows = getattr(batch, "adapter_rows", None)
    if lora is None or rows is None:
        return
    if x.is_cuda and y.dtype == torch.bfloat16:
        ads = {s: ad.weights[module] for s, ad in lora.slots.items() if module in ad.weights}
        if ads:
            from .ops import cuda as K
            n = next(iter(ads.values()))[1].shape[0] if cols is None else cols
            K.lora_bgmv(x, rows, ads, {s: lora.slots[s].scaling for s in ads}, y, col0, n)
        return
    d = lora.delta(module, x, rows)
    if d is not None:
        n = d.shape[1] if cols is None else cols
        y[:, col0:col0 + n] += d.to(y.dtype)
