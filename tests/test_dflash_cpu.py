"""Block-diffusion drafter: the paged, one-pass block forward against a dense restatement, and the engine loop with
the drafter attached (greedy speculative decoding must reproduce plain greedy decoding token for token)."""
import math

import torch

from atlas_b200.config import EngineConfig, tiny_dense
from atlas_b200.engine import LLMEngine
from atlas_b200.models import build_model
from atlas_b200.models.dflash import BlockDiffusionDrafter, DFlashConfig
from atlas_b200.ops import reference as ref
from atlas_b200.sampling import SamplingParams


def _drafter(model, layers=(0, 1)):
    dcfg = DFlashConfig(hidden_size=model.cfg.hidden_size, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=32, block_len=5, target_layer_ids=list(layers))
    return BlockDiffusionDrafter(dcfg, model).init_random(1)


def _rope(x, pos, cache, d):
    half = d // 2
    cos, sin = cache[pos.long(), :half][:, None, :], cache[pos.long(), half:][:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def test_block_forward_matches_dense_restatement():
    torch.manual_seed(0)
    model = build_model(tiny_dense("float32"), device="cpu").init_random(0)
    d = _drafter(model)
    d.alloc_cache(16, 16)
    d.finalize(256)
    ctx, k = 21, 4
    table = [3, 7, 1]
    H = model.cfg.hidden_size
    aux = [torch.randn(ctx, H), torch.randn(ctx, H)]
    feats = d.context_features(aux)
    pos = torch.arange(ctx, dtype=torch.int32)
    slots = torch.tensor([table[p // 16] * 16 + p % 16 for p in range(ctx)], dtype=torch.int32)
    d.add_context(feats, pos, slots)
    got = d.propose([17], [ctx], [table], k)[0]

    # dense restatement: keys / values of [context features ; block states], no mask
    eps, g = d.cfg.rms_norm_eps, k + 1
    x = d.mask_embed.repeat(g, 1).clone()
    x[0] = d.embed(torch.tensor([17]))[0]
    bpos = torch.arange(ctx, ctx + g, dtype=torch.int32)
    for l in d.layers:
        h = _rms(x, l.input_norm, eps)
        q = (h @ l.q.weight.t()).view(g, l.hq, l.d)
        src = torch.cat([feats, h])
        kv = src @ l.kv.weight.t()
        kk = kv[:, :l.hkv * l.d].view(-1, l.hkv, l.d)
        vv = kv[:, l.hkv * l.d:].view(-1, l.hkv, l.d)
        q = _rope(_rms(q, l.q_norm, eps), bpos, d.rope_cache, l.d)
        kk = _rope(_rms(kk, l.k_norm, eps), torch.cat([pos, bpos]), d.rope_cache, l.d)
        rep = l.hq // l.hkv
        s = torch.einsum("qhd,khd->hqk", q, kk.repeat_interleave(rep, 1)) / math.sqrt(l.d)
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv.repeat_interleave(rep, 1)).reshape(g, -1)
        x = x + a @ l.o.weight.t()
        h2 = _rms(x, l.post_norm, eps)
        gu = h2 @ l.mlp.gate_up.weight.t()
        i = gu.shape[-1] // 2
        x = x + (torch.nn.functional.silu(gu[:, :i]) * gu[:, i:]) @ l.mlp.down.weight.t()
    y = _rms(x, d.final_norm, eps)
    want = model.compute_logits(y[1:]).argmax(-1).tolist()
    assert got == want


def test_engine_with_drafter_is_lossless_under_greedy():
    model = build_model(tiny_dense("float32"), device="cpu").init_random(0)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, model.cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 33, 18)]
    sp = SamplingParams(max_tokens=14, temperature=0.0, ignore_eos=True)
    base = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=4, max_seq_len=128, max_prefill_tokens=32,
                                         enable_prefix_caching=False)).generate(prompts, sp)
    model.dflash = _drafter(model)
    eng = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=4, max_seq_len=128, max_prefill_tokens=32,
                                        enable_prefix_caching=False, speculative=True, num_drafts=4, mtp_gate=False))
    out = eng.generate(prompts, sp)
    assert [o.output_tokens for o in out] == [o.output_tokens for o in base]
    assert eng.spec.proposed_steps > 0 and eng.stats.spec_proposed > 0
    model.dflash, model.capture_layers = None, ()


def test_drafter_checkpoint_round_trip(tmp_path):
    from safetensors.torch import save_file
    model = build_model(tiny_dense("float32"), device="cpu").init_random(0)
    a = _drafter(model)
    t = {"fc.weight": a.fc.weight, "hidden_norm.weight": a.feat_norm * 1.5, "norm.weight": a.final_norm * 0.5,
         "mask_embed": a.mask_embed}
    for i, l in enumerate(a.layers):
        p = f"layers.{i}."
        hk = l.hkv * l.d
        inter = l.mlp.gate_up.weight.shape[0] // 2
        t.update({p + "self_attn.q_proj.weight": l.q.weight, p + "self_attn.k_proj.weight": l.kv.weight[:hk],
                  p + "self_attn.v_proj.weight": l.kv.weight[hk:], p + "self_attn.o_proj.weight": l.o.weight,
                  p + "self_attn.q_norm.weight": l.q_norm, p + "self_attn.k_norm.weight": l.k_norm,
                  p + "input_layernorm.weight": l.input_norm, p + "post_attention_layernorm.weight": l.post_norm,
                  p + "mlp.gate_proj.weight": l.mlp.gate_up.weight[:inter], p + "mlp.up_proj.weight": l.mlp.gate_up.weight[inter:],
                  p + "mlp.down_proj.weight": l.mlp.down.weight})
    save_file({k: v.contiguous().clone() for k, v in t.items()}, str(tmp_path / "model.safetensors"))
    b = BlockDiffusionDrafter(a.dcfg, model).load(str(tmp_path))
    a.feat_norm, a.final_norm = a.feat_norm * 1.5, a.final_norm * 0.5
    for d in (a, b):
        d.alloc_cache(8, 16)
        d.finalize(128)
    H = model.cfg.hidden_size
    aux = [torch.randn(10, H), torch.randn(10, H)]
    pos = torch.arange(10, dtype=torch.int32)
    outs = []
    for d in (a, b):
        d.add_context(d.context_features(aux), pos, pos + 16)
        outs.append(d.propose([5], [10], [[1, 2]], 4))
    assert outs[0] == outs[1]
