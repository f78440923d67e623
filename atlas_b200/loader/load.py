"""HF checkpoint -> model: weight names of the supported families, fusion (QKV, gate|up, GDN in-projection
de-interleave), tensor / expert parallel sharding and quantised-format pass-through.

Sharding happens on the checkpoint tensors (quantised ones are sliced together with their scales, high-precision
ones are sliced first and quantised afterwards when the configuration asks for it).

Reference parity: ``crates/spark-model/src/weight_loader/{qwen3,qwen35,qwen35_dense,mistral}.rs``,
``weight_map/*``, ``tp_shard.rs``, ``factory.rs:68`` (``loader_for_config``).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from ..config import ModelConfig
from ..layers import ParallelCtx
from ..layers.moe import ExpertWeights
from ..models import DecoderLM, build_model
from ..models.decoder import quant_kinds
from ..ops import LinearWeight
from .checkpoint import Checkpoint
from .qtensor import QTensor, as_q, cat_rows, to_linear


def load_model(path: str, pctx: Optional[ParallelCtx] = None, device="cpu", dtype: Optional[str] = None,
               max_pos: Optional[int] = None, with_mtp: Optional[bool] = None) -> DecoderLM:
    gguf_path = _gguf_file(path)
    if gguf_path is not None:
        from .gguf import load_gguf_model
        return load_gguf_model(gguf_path, pctx, device=device, dtype=dtype, max_pos=max_pos)
    cfg = ModelConfig.from_pretrained(path)
    if dtype:
        cfg.dtype = dtype
    model = build_model(cfg, pctx, device=device, with_mtp=with_mtp)
    load_weights(model, Checkpoint(path))
    model.finalize(max_pos)
    return model


def _gguf_file(path: str) -> Optional[str]:
    """``path`` itself when it is a ``.gguf`` file, or the single ``.gguf`` inside a directory without ``config.json``."""
    if os.path.isfile(path) and path.endswith(".gguf"):
        return path
    if os.path.isdir(path) and not os.path.exists(os.path.join(path, "config.json")):
        found = sorted(f for f in os.listdir(path) if f.endswith(".gguf"))
        if len(found) == 1:
            return os.path.join(path, found[0])
    return None


def _vec(ck: Checkpoint, name: str, model: DecoderLM, dtype=None) -> Optional[torch.Tensor]:
    t = ck.maybe(name)
    return None if t is None else t.to(device=model.device, dtype=dtype or model.dtype).contiguous()


def _lin(q: QTensor, kind: str, model: DecoderLM, bias=None) -> LinearWeight:
    return to_linear(q.to(model.device), kind, model.dtype, bias)


def _load_attention(ck, pre, mixer, model, kind) -> None:
    cfg, tp, r = mixer.cfg, mixer.pctx.tp_size, mixer.pctx.tp_rank
    d = mixer.d
    q, k, v, o = (ck.linear(f"{pre}.{n}_proj") for n in "qkvo")
    if mixer.gated:
        heads = range(r * mixer.hq, (r + 1) * mixer.hq)
        qp = cat_rows([q.rows(h * 2 * d, h * 2 * d + d) for h in heads])
        gp = cat_rows([q.rows(h * 2 * d + d, (h + 1) * 2 * d) for h in heads])
    else:
        qp, gp = q.rows(r * mixer.hq * d, (r + 1) * mixer.hq * d), None
    kv0 = ((r // mixer.kv_rep) * mixer.hkv) * d if tp > 1 else 0
    kp, vp = k.rows(kv0, kv0 + mixer.hkv * d), v.rows(kv0, kv0 + mixer.hkv * d)
    bias = None
    if ck.has(f"{pre}.q_proj.bias"):
        bq, bk, bv = (ck.get(f"{pre}.{n}_proj.bias") for n in "qkv")
        bias = torch.cat([bq[r * mixer.hq * d:(r + 1) * mixer.hq * d], bk[kv0:kv0 + mixer.hkv * d],
                          bv[kv0:kv0 + mixer.hkv * d]]).to(device=model.device, dtype=model.dtype)
    parts = [qp, kp, vp] + ([gp] if gp is not None else [])
    mixer.qkv = _lin(cat_rows(parts), kind, model, bias)
    mixer.o = _lin(o.cols(r * mixer.hq * d, (r + 1) * mixer.hq * d), kind, model)
    mixer.q_norm = _vec(ck, f"{pre}.q_norm.weight", model)
    mixer.k_norm = _vec(ck, f"{pre}.k_norm.weight", model)


def _load_mla(ck, pre, mixer, model, kind) -> None:
    """Latent attention: the rope rows of ``q_b`` / ``kv_a`` are reordered and moved in front of the nope rows, which
    crosses the 128-row scale blocks of a block-quantised checkpoint, so these (small) projections are dequantised
    and quantised again in the loaded layout."""
    dq = lambda n: ck.linear(f"{pre}.{n}").dequant().float()
    has_qa = ck.has(f"{pre}.q_a_proj.weight")
    q_a = dq("q_a_proj") if has_qa else None
    q_b = dq("q_b_proj") if has_qa else dq("q_proj")
    norm = lambda n: ck.get(f"{pre}.{n}.weight").to(device=model.device, dtype=model.dtype).contiguous()
    cast = lambda t: None if t is None else t.to(device=model.device, dtype=model.dtype)
    mixer.load(cast(q_a), norm("q_a_layernorm") if has_qa else None, cast(q_b), cast(dq("kv_a_proj_with_mqa")),
               norm("kv_a_layernorm"), cast(dq("kv_b_proj")), cast(dq("o_proj")), mixer.cfg.rope_interleaved)


def _load_mlp(ck, pre, mlp, model, kind) -> None:
    tp, r = (mlp.pctx.tp_size, mlp.pctx.tp_rank) if mlp.shard else (1, 0)
    g, u, dn = (ck.linear(f"{pre}.{n}_proj") for n in ("gate", "up", "down"))
    s = mlp.inter // tp
    mlp.gate_up = _lin(cat_rows([g.rows(r * s, (r + 1) * s), u.rows(r * s, (r + 1) * s)]), kind, model)
    mlp.down = _lin(dn.cols(r * s, (r + 1) * s), kind, model)


def _stack_gscale(parts: List[QTensor]) -> torch.Tensor:
    """``[E]`` when every expert has one global scale, ``[E,N]`` when fused rows carry their own."""
    if all(p.gscale.numel() == 1 for p in parts):
        return torch.cat([p.gscale.float().reshape(1) for p in parts])
    return torch.stack([p.gscale.float().reshape(-1).expand(p.weight.shape[0]) for p in parts])


def _stack_experts(parts13: List[QTensor], parts2: List[QTensor], want_kind: str, model) -> ExpertWeights:
    kinds = {p.kind for p in parts13 + parts2}
    dev = model.device
    if kinds == {"fp8_block"}:
        return ExpertWeights("fp8_block", torch.stack([p.weight for p in parts13]).to(dev), torch.stack([p.weight for p in parts2]).to(dev),
                             torch.stack([p.scale.float() for p in parts13]).to(dev), torch.stack([p.scale.float() for p in parts2]).to(dev))
    if kinds == {"nvfp4"}:
        return ExpertWeights("nvfp4", torch.stack([p.weight for p in parts13]).to(dev), torch.stack([p.weight for p in parts2]).to(dev),
                             torch.stack([p.scale for p in parts13]).to(dev), torch.stack([p.scale for p in parts2]).to(dev),
                             _stack_gscale(parts13).to(dev), _stack_gscale(parts2).to(dev))
    w13 = torch.stack([p.dequant().to(model.dtype) for p in parts13]).to(dev)
    w2 = torch.stack([p.dequant().to(model.dtype) for p in parts2]).to(dev)
    return ExpertWeights.from_dense(w13, w2, want_kind)


def _load_moe(ck, pre, moe, model, dense_kind, expert_kind) -> None:
    router = ck.get(f"{pre}.gate.weight")
    moe.router = LinearWeight("dense", router.to(device=model.device, dtype=model.dtype).contiguous())
    p13, p2 = [], []
    for e in range(moe.e_lo, moe.e_hi):
        g, u, dn = (ck.linear(f"{pre}.experts.{e}.{n}_proj") for n in ("gate", "up", "down"))
        p13.append(cat_rows([g, u]))
        p2.append(as_q(dn))
    moe.experts = _stack_experts(p13, p2, expert_kind, model)
    bias = ck.maybe(f"{pre}.gate.e_score_correction_bias")
    if bias is not None:
        moe.router_bias = bias.float().to(model.device).contiguous()
    if moe.shared is not None:
        shared = "shared_experts" if ck.has(f"{pre}.shared_experts.gate_proj.weight") else "shared_expert"
        _load_mlp(ck, f"{pre}.{shared}", moe.shared, model, dense_kind)
        sg = ck.maybe(f"{pre}.shared_expert_gate.weight")
        moe.shared_gate = None if sg is None else sg.to(device=model.device, dtype=model.dtype)


def _load_gdn(ck, pre, mixer, model, kind) -> None:
    """The qkvz / ba projections may be quantised; the row regrouping is done on QTensors (128-aligned segments stay
    quantised, the tiny b/a rows fall back to high precision inside ``cat_rows`` if needed)."""
    cfg, tp, r = mixer.cfg, mixer.pctx.tp_size, mixer.pctx.tp_rank
    HK, HV, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, mixer.dk, mixer.dv
    rep = HV // HK
    if ck.has(f"{pre}.in_proj_qkv.weight"):
        # Qwen3.5 layout: flat [q | k | v] rows plus separate z, b and a projections (value head i pairs with key head
        # i // rep, so a rank's heads are contiguous row ranges)
        qkv, zp = ck.linear(f"{pre}.in_proj_qkv"), ck.linear(f"{pre}.in_proj_z")
        bp, ap = ck.linear(f"{pre}.in_proj_b"), ck.linear(f"{pre}.in_proj_a")
        KDf, kd, vd, hv_n = HK * dk, mixer.kd, mixer.vd, mixer.hv
        main = cat_rows([qkv.rows(r * kd, (r + 1) * kd), qkv.rows(KDf + r * kd, KDf + (r + 1) * kd),
                         qkv.rows(2 * KDf + r * vd, 2 * KDf + (r + 1) * vd), zp.rows(r * vd, (r + 1) * vd)])
        tail = cat_rows([bp.rows(r * hv_n, (r + 1) * hv_n), ap.rows(r * hv_n, (r + 1) * hv_n)])
    else:
        qkvz, ba = ck.linear(f"{pre}.in_proj_qkvz"), ck.linear(f"{pre}.in_proj_ba")
        grp = 2 * dk + 2 * rep * dv
        heads = range(r * mixer.hk, (r + 1) * mixer.hk)
        seg = lambda lo, hi: [qkvz.rows(h * grp + lo, h * grp + hi) for h in heads]
        qs, ks = seg(0, dk), seg(dk, 2 * dk)
        vs, zs = seg(2 * dk, 2 * dk + rep * dv), seg(2 * dk + rep * dv, grp)
        bs = [ba.rows(h * 2 * rep, h * 2 * rep + rep) for h in heads]
        as_ = [ba.rows(h * 2 * rep + rep, (h + 1) * 2 * rep) for h in heads]
        main = cat_rows(qs + ks + vs + zs)
        tail = cat_rows(bs + as_)
    if main.kind == "fp8_block" and main.weight.shape[0] % 128 == 0 and tail.kind == "fp8_block":
        fused = cat_rows([main, tail])
    elif main.kind == tail.kind == "dense":
        fused = cat_rows([main, tail])
    else:
        fused = QTensor("dense", torch.cat([main.dequant().float(), tail.dequant().float()], 0))
    mixer.in_proj = _lin(fused, kind, model)
    cw = ck.get(f"{pre}.conv1d.weight")
    cw = cw.reshape(cw.shape[0], -1)
    KD, VD = HK * dk, HV * dv
    sk, sv = slice(r * mixer.kd, (r + 1) * mixer.kd), slice(r * mixer.vd, (r + 1) * mixer.vd)
    mixer.conv_w = torch.cat([cw[:KD][sk], cw[KD:2 * KD][sk], cw[2 * KD:2 * KD + VD][sv]], 0).to(device=model.device, dtype=model.dtype).contiguous()
    hv = slice(r * mixer.hv, (r + 1) * mixer.hv)
    mixer.dt_bias = ck.get(f"{pre}.dt_bias")[hv].float().to(model.device).contiguous()
    mixer.A_log = ck.get(f"{pre}.A_log")[hv].float().to(model.device).contiguous()
    mixer.norm_w = _vec(ck, f"{pre}.norm.weight", model)
    mixer.out_proj = _lin(ck.linear(f"{pre}.out_proj").cols(r * mixer.vd, (r + 1) * mixer.vd), kind, model)


def _load_layer(ck, pre, layer, model, dense_kind, expert_kind) -> None:
    layer.input_norm = _vec(ck, f"{pre}.input_layernorm.weight", model)
    layer.post_norm = _vec(ck, f"{pre}.post_attention_layernorm.weight", model)
    if layer.cfg.sandwich_norms:
        layer.pre_ffn_norm = _vec(ck, f"{pre}.pre_feedforward_layernorm.weight", model)
        layer.post_ffn_norm = _vec(ck, f"{pre}.post_feedforward_layernorm.weight", model)
    if layer.kind == "attention" and layer.cfg.kv_lora_rank > 0:
        _load_mla(ck, f"{pre}.self_attn", layer.mixer, model, dense_kind)
    elif layer.kind == "attention":
        _load_attention(ck, f"{pre}.self_attn", layer.mixer, model, dense_kind)
    else:
        _load_gdn(ck, f"{pre}.linear_attn", layer.mixer, model, dense_kind)
    if layer.is_moe:
        _load_moe(ck, f"{pre}.mlp", layer.ffn, model, dense_kind, expert_kind)
    else:
        _load_mlp(ck, f"{pre}.mlp", layer.ffn, model, dense_kind)


def _load_mamba2(ck, pre, mixer, model, kind) -> None:
    """HF ``mixer.in_proj`` rows are ``[z | x | B | C | dt]`` over all heads / groups; the rank's slices are cut on the
    (possibly quantised) tensor and re-fused."""
    cfg, r = mixer.cfg, mixer.pctx.tp_rank
    HP, GN, Hh = cfg.mamba_num_heads * cfg.mamba_head_dim, cfg.mamba_n_groups * cfg.ssm_state_size, cfg.mamba_num_heads
    di, gn, hh = mixer.d_inner, mixer.g * mixer.n, mixer.h
    inp = ck.linear(f"{pre}.in_proj")
    offs = [0, HP, 2 * HP, 2 * HP + GN, 2 * HP + 2 * GN]
    sizes = [di, di, gn, gn, hh]
    parts = [inp.rows(o + r * n, o + (r + 1) * n) for o, n in zip(offs, sizes)]
    fused = cat_rows(parts)
    mixer.in_proj = _lin(fused, kind, model)
    cw = ck.get(f"{pre}.conv1d.weight")
    cw = cw.reshape(cw.shape[0], -1)
    cut = lambda t: torch.cat([t[o + r * n:o + (r + 1) * n] for o, n in zip([0, HP, HP + GN], [di, gn, gn])], 0)
    mixer.conv_w = cut(cw).to(device=model.device, dtype=model.dtype).contiguous()
    cb = ck.maybe(f"{pre}.conv1d.bias")
    mixer.conv_b = None if cb is None else cut(cb).to(device=model.device, dtype=model.dtype).contiguous()
    hs = slice(r * hh, (r + 1) * hh)
    mixer.A_log = ck.get(f"{pre}.A_log")[hs].float().to(model.device).contiguous()
    mixer.D = ck.get(f"{pre}.D")[hs].float().to(model.device).contiguous()
    mixer.dt_bias = ck.get(f"{pre}.dt_bias")[hs].float().to(model.device).contiguous()
    mixer.norm_w = ck.get(f"{pre}.norm.weight")[r * di:(r + 1) * di].to(device=model.device, dtype=model.dtype).contiguous()
    mixer.out_proj = _lin(ck.linear(f"{pre}.out_proj").cols(r * di, (r + 1) * di), kind, model)


def _load_single_blocks(model: DecoderLM, ck: Checkpoint, dense_kind: str) -> None:
    """Nemotron-H naming: ``backbone.embeddings``, ``backbone.layers.N.{norm, mixer.*}``, ``backbone.norm_f``."""
    root = "backbone" if any(k.startswith("backbone.") for k in ck.keys()) else "model"
    emb = ck.maybe(f"{root}.embeddings.weight")
    if emb is None:
        emb = ck.get(f"{root}.embedding.weight")            # spelling of the original checkpoints
    model.embed = emb.to(device=model.device, dtype=model.dtype)
    for i, blk in enumerate(model.layers):
        pre = f"{root}.layers.{i}"
        blk.input_norm = _vec(ck, f"{pre}.norm.weight", model)
        if blk.kind == "mamba2":
            _load_mamba2(ck, f"{pre}.mixer", blk.mixer, model, dense_kind)
        elif blk.kind == "attention":
            _load_attention(ck, f"{pre}.mixer", blk.mixer, model, dense_kind)
        else:
            mlp = blk.ffn
            tp, r = (mlp.pctx.tp_size, mlp.pctx.tp_rank) if mlp.shard else (1, 0)
            s = mlp.inter // tp
            mlp.gate_up = _lin(ck.linear(f"{pre}.mixer.up_proj").rows(r * s, (r + 1) * s), dense_kind, model)
            mlp.down = _lin(ck.linear(f"{pre}.mixer.down_proj").cols(r * s, (r + 1) * s), dense_kind, model)
    model.final_norm = _vec(ck, f"{root}.norm_f.weight", model)
    head = ck.maybe("lm_head.weight")
    if head is None or model.cfg.tie_word_embeddings:
        head = model.embed
    model.set_lm_head(head.to(device=model.device, dtype=model.dtype))
    model.mtp = None
    ck.close()


def load_weights(model: DecoderLM, ck: Checkpoint) -> None:
    cfg = model.cfg
    dense_kind, expert_kind = quant_kinds(cfg)
    if cfg.block_types:
        if any(k.endswith((".weight_scale_inv", ".weight_scale", ".weight_packed")) for k in ck.keys()):
            dense_kind = "dense"
        return _load_single_blocks(model, ck, dense_kind)
    if any(k.endswith((".weight_scale_inv", ".weight_scale", ".weight_packed")) for k in ck.keys()):
        # a pre-quantised checkpoint: what it left in high precision (its ignore list) stays in high precision
        dense_kind = expert_kind = "dense"
    root = "model" if any(k.startswith("model.layers.") for k in ck.keys()) else "model.language_model"
    if not ck.has(f"{root}.embed_tokens.weight"):
        # multimodal wrappers nest the text model under further prefixes: take whatever precedes the embedding table
        root = next(k[:-len(".embed_tokens.weight")] for k in ck.keys() if k.endswith(".embed_tokens.weight") and "mtp" not in k)
    model.embed = ck.get(f"{root}.embed_tokens.weight").to(device=model.device, dtype=model.dtype)
    for i, layer in enumerate(model.layers):
        _load_layer(ck, f"{root}.layers.{i}", layer, model, dense_kind, expert_kind)
    model.final_norm = _vec(ck, f"{root}.norm.weight", model)
    vis = next((k[:-len("patch_embed.proj.weight")] for k in ck.keys() if k.endswith("visual.patch_embed.proj.weight")), None)
    if cfg.vision is not None and vis is not None:
        from ..models.vision import VisionTower
        model.vision = VisionTower(cfg.vision, model.device, model.dtype).load(ck.get, vis)
    head = ck.maybe("lm_head.weight")
    if head is None or cfg.tie_word_embeddings:
        head = model.embed
    model.set_lm_head(head.to(device=model.device, dtype=model.dtype))
    if model.mtp is not None and ck.has("mtp.fc.weight"):
        m = model.mtp
        m.fc = LinearWeight("dense", ck.get("mtp.fc.weight").to(device=model.device, dtype=model.dtype).contiguous())
        m.norm_e = _vec(ck, "mtp.pre_fc_norm_embedding.weight", model)
        m.norm_h = _vec(ck, "mtp.pre_fc_norm_hidden.weight", model)
        m.final_norm = _vec(ck, "mtp.norm.weight", model)
        _load_layer(ck, "mtp.layers.0", m.layer, model, dense_kind, expert_kind)
    elif model.mtp is not None:
        model.mtp = None          # the checkpoint ships no draft head
    ck.close()
