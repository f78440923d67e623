"""Checkpoint loader parity: a tiny random HF model saved with ``save_pretrained`` and read back through the loader
must give the same logits as the ``transformers`` implementation (fp32, CPU), for every supported family, with and
without tensor / expert parallel sharding, and for pre-quantised (FP8 block scale, NVFP4) checkpoints."""
import json
import os

import pytest
import torch

from atlas_b200 import quant as Q
from atlas_b200.config import ModelConfig
from atlas_b200.layers import ParallelCtx
from atlas_b200.loader import Checkpoint, QTensor, load_model
from atlas_b200.loader.qtensor import cat_rows
from atlas_b200.parallel.comm import FakeWorld

transformers = pytest.importorskip("transformers")


def _hf(kind: str):
    torch.manual_seed(0)
    common = dict(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  head_dim=64, max_position_embeddings=256, rms_norm_eps=1e-6, tie_word_embeddings=False)
    if kind == "llama":
        cfg = transformers.LlamaConfig(intermediate_size=512, rope_theta=10000.0, **common)
        m = transformers.LlamaForCausalLM(cfg)
    elif kind == "qwen2":
        cfg = transformers.Qwen2Config(intermediate_size=512, **{k: v for k, v in common.items() if k != "head_dim"})
        m = transformers.Qwen2ForCausalLM(cfg)
    elif kind == "qwen3":
        cfg = transformers.Qwen3Config(intermediate_size=512, **common)
        m = transformers.Qwen3ForCausalLM(cfg)
    elif kind == "qwen3_moe":
        cfg = transformers.Qwen3MoeConfig(intermediate_size=512, moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                                          norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], **common)
        m = transformers.Qwen3MoeForCausalLM(cfg)
    elif kind == "qwen3_next":
        cfg = transformers.Qwen3NextConfig(intermediate_size=512, moe_intermediate_size=128, shared_expert_intermediate_size=128,
                                           num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
                                           mlp_only_layers=[], linear_num_key_heads=2, linear_num_value_heads=4,
                                           linear_key_head_dim=64, linear_value_head_dim=64, linear_conv_kernel_dim=4,
                                           partial_rotary_factor=0.25, layer_types=["linear_attention", "full_attention"],
                                           **common)
        m = transformers.Qwen3NextForCausalLM(cfg)
    elif kind == "qwen3_5":
        cfg = transformers.Qwen3_5TextConfig(intermediate_size=512, linear_num_key_heads=2, linear_num_value_heads=4,
                                             linear_key_head_dim=64, linear_value_head_dim=64, linear_conv_kernel_dim=4,
                                             layer_types=["linear_attention", "full_attention"], **common)
        m = transformers.Qwen3_5ForCausalLM(cfg)
    elif kind == "qwen3_5_moe":
        cfg = transformers.Qwen3_5MoeTextConfig(moe_intermediate_size=128, shared_expert_intermediate_size=128, num_experts=8,
                                                num_experts_per_tok=2, linear_num_key_heads=2, linear_num_value_heads=4,
                                                linear_key_head_dim=64, linear_value_head_dim=64, linear_conv_kernel_dim=4,
                                                layer_types=["linear_attention", "full_attention"], **common)
        m = transformers.Qwen3_5MoeForCausalLM(cfg)
    elif kind == "deepseek_v3":
        cfg = transformers.DeepseekV3Config(vocab_size=512, hidden_size=256, num_hidden_layers=3, num_attention_heads=4,
                                            num_key_value_heads=4, intermediate_size=512, moe_intermediate_size=128,
                                            n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, n_group=4, topk_group=2,
                                            first_k_dense_replace=1, kv_lora_rank=64, q_lora_rank=96, qk_nope_head_dim=32,
                                            qk_rope_head_dim=16, v_head_dim=32, max_position_embeddings=256,
                                            routed_scaling_factor=2.5, norm_topk_prob=True, tie_word_embeddings=False)
        m = transformers.DeepseekV3ForCausalLM(cfg)
        with torch.no_grad():
            for n, b in m.named_buffers():
                if n.endswith("e_score_correction_bias"):
                    b.copy_(torch.rand_like(b) * 0.2)
    elif kind == "gemma3":
        cfg = transformers.Gemma3TextConfig(vocab_size=512, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                                            num_key_value_heads=2, head_dim=64, intermediate_size=512, sliding_window=8,
                                            max_position_embeddings=256, query_pre_attn_scalar=96,
                                            layer_types=["sliding_attention", "sliding_attention", "full_attention",
                                                         "sliding_attention"], final_logit_softcapping=20.0,
                                            tie_word_embeddings=True)
        m = transformers.Gemma3ForCausalLM(cfg)
    elif kind == "nemotron_h":
        cfg = transformers.NemotronHConfig(vocab_size=512, hidden_size=256, layers_block_type=["mamba", "attention", "mamba", "mamba"],
                                           num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=512,
                                           mamba_num_heads=8, mamba_head_dim=32, ssm_state_size=32, n_groups=2, conv_kernel=4,
                                           chunk_size=64, max_position_embeddings=256, tie_word_embeddings=False,
                                           use_mamba_kernels=False)
        # chunk_size covers the whole test sequence: the eager fallback of the oracle passes state between chunks
        # inexactly (its output moves by ~1e-3 with the chunk size), a single chunk is the exact recurrence
        m = transformers.NemotronHForCausalLM(cfg)
    else:
        raise ValueError(kind)
    m = m.float().eval()
    with torch.no_grad():                      # make norms / biases non-trivial
        for n, p in m.named_parameters():
            if n.endswith("norm.weight") or n.endswith("layernorm.weight") or n.endswith("norm_f.weight"):
                p.add_(torch.randn_like(p) * 0.1)
            elif n.endswith(".bias"):
                p.copy_(torch.randn_like(p) * 0.1)
    return m


def _save(m, path):
    m.save_pretrained(path, safe_serialization=True)
    return str(path)


def _ours_logits(model, toks):
    return model.forward_dense_reference(toks)


@pytest.mark.parametrize("kind", ["llama", "qwen2", "qwen3", "qwen3_moe", "qwen3_next", "qwen3_5", "qwen3_5_moe", "nemotron_h", "deepseek_v3", "gemma3"])
def test_logits_match_transformers(kind, tmp_path):
    hf = _hf(kind)
    path = _save(hf, tmp_path)
    toks = torch.randint(0, 512, (24,), generator=torch.Generator().manual_seed(3)).tolist()
    with torch.no_grad():
        want = hf(torch.tensor([toks])).logits[0]
    model = load_model(path, dtype="float32", with_mtp=False)
    got = _ours_logits(model, toks)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=1e-3)


@pytest.mark.parametrize("kind", ["qwen3", "qwen3_next", "qwen3_5", "nemotron_h", "deepseek_v3", "gemma3"])
def test_sharded_load_matches_full(kind, tmp_path):
    """TP=2 (dense) / TP=2+EP=2 (hybrid MoE): the ranks, run in lock-step over the in-process fake communicator,
    reproduce the single-rank logits."""
    hf = _hf(kind)
    path = _save(hf, tmp_path)
    toks = torch.randint(0, 512, (12,), generator=torch.Generator().manual_seed(4)).tolist()
    full = _ours_logits(load_model(path, dtype="float32", with_mtp=False), toks)
    world = FakeWorld(2, timeout_s=60.0)

    def rank_fn(r):
        comm = world.comm(r)
        pctx = ParallelCtx(tp_rank=r, tp_size=2, ep_rank=r, ep_size=2, comm=comm, ep_comm=comm)
        model = load_model(path, pctx, dtype="float32", with_mtp=False)
        return _ours_logits(model, toks)

    outs = world.run(rank_fn)
    for o in outs:
        torch.testing.assert_close(o, full, atol=2e-4, rtol=1e-3)


def _requantise_checkpoint(src, dst, fmt):
    """Rewrite every 2-D projection weight of a saved checkpoint in a quantised on-disk format."""
    from safetensors.torch import load_file, save_file
    os.makedirs(dst, exist_ok=True)
    tensors = load_file(os.path.join(src, "model.safetensors"))
    out = {}
    for name, t in tensors.items():
        is_proj = name.endswith("_proj.weight") and t.dim() == 2 and t.shape[1] % 128 == 0 and t.shape[0] % 128 == 0
        if not is_proj:
            out[name] = t
            continue
        base = name[:-len(".weight")]
        if fmt == "fp8":
            q, s = Q.quantize_fp8_block(t.float())
            out[name], out[base + ".weight_scale_inv"] = q, s
        elif fmt == "modelopt":
            p, s, g = Q.quantize_nvfp4(t.float())
            out[name], out[base + ".weight_scale"], out[base + ".weight_scale_2"] = p, s, g.reshape(())
        else:   # compressed-tensors
            p, s, g = Q.quantize_nvfp4(t.float())
            out[base + ".weight_packed"], out[base + ".weight_scale"] = p, s
            out[base + ".weight_global_scale"] = (1.0 / g).reshape(1)
    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(dst, "model.safetensors"))
    cfg = json.load(open(os.path.join(src, "config.json")))
    if fmt == "fp8":
        cfg["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128]}
    elif fmt == "modelopt":
        cfg["quantization_config"] = {"quant_method": "modelopt", "quant_algo": "NVFP4"}
    else:
        cfg["quantization_config"] = {"quant_method": "compressed-tensors", "format": "nvfp4-pack-quantized"}
    json.dump(cfg, open(os.path.join(dst, "config.json"), "w"))
    return dst


@pytest.mark.parametrize("kind,fmt", [("qwen3", "fp8"), ("qwen3", "modelopt"), ("qwen3", "compressed"),
                                      ("qwen3_moe", "modelopt"), ("qwen3_next", "modelopt")])
def test_prequantised_checkpoint_roundtrip(kind, fmt, tmp_path):
    """A pre-quantised checkpoint keeps its codes and scales bit-for-bit through slicing / fusing, and its logits
    match the dequantised weights run through ``transformers``."""
    hf = _hf(kind)
    src = _save(hf, tmp_path / "src")
    dst = _requantise_checkpoint(src, str(tmp_path / fmt), fmt)
    model = load_model(dst, dtype="float32", with_mtp=False)
    want_kind = "fp8_block" if fmt == "fp8" else "nvfp4"
    if kind == "qwen3":
        assert model.layers[0].mixer.qkv.kind == want_kind and model.layers[0].ffn.down.kind == want_kind
    else:
        assert model.layers[0].ffn.experts.kind == want_kind
    # oracle: transformers on a checkpoint holding the dequantised weights
    from safetensors.torch import load_file, save_file
    ck = Checkpoint(dst)
    deq = str(tmp_path / "deq")
    os.makedirs(deq)
    dense = {}
    for name, t in load_file(os.path.join(src, "model.safetensors")).items():
        dense[name] = ck.linear(name[:-len(".weight")]).dequant().float().contiguous() if name.endswith("_proj.weight") else t
    save_file(dense, os.path.join(deq, "model.safetensors"))
    with open(os.path.join(src, "config.json")) as f, open(os.path.join(deq, "config.json"), "w") as g:
        g.write(f.read())
    hf = transformers.AutoModelForCausalLM.from_pretrained(deq, torch_dtype=torch.float32).eval()
    toks = torch.randint(0, 512, (16,), generator=torch.Generator().manual_seed(5)).tolist()
    with torch.no_grad():
        want = hf(torch.tensor([toks])).logits[0]
    got = _ours_logits(model, toks)
    # activations are quantised per 128 on the fp8 path; NVFP4 weights run against full-precision activations
    tol = dict(atol=0.08, rtol=0.05) if fmt == "fp8" else dict(atol=2e-4, rtol=1e-3)
    torch.testing.assert_close(got, want, **tol)


def test_qtensor_slices_are_exact():
    w = torch.randn(512, 384)
    q, s = Q.quantize_fp8_block(w)
    qt = QTensor("fp8_block", q, s)
    full = qt.dequant()
    torch.testing.assert_close(qt.rows(128, 384).dequant(), full[128:384], atol=0, rtol=0)
    torch.testing.assert_close(qt.cols(128, 256).dequant(), full[:, 128:256], atol=0, rtol=0)
    torch.testing.assert_close(qt.rows(64, 96).dequant(), full[64:96], atol=0, rtol=0)
    torch.testing.assert_close(cat_rows([qt.rows(0, 128), qt.rows(256, 512)]).dequant(),
                               torch.cat([full[:128], full[256:]]), atol=0, rtol=0)
    p, sc, g = Q.quantize_nvfp4(w)
    nt = QTensor("nvfp4", p, sc, g)
    nfull = nt.dequant()
    torch.testing.assert_close(nt.rows(10, 70).dequant(), nfull[10:70], atol=0, rtol=0)
    torch.testing.assert_close(nt.cols(32, 160).dequant(), nfull[:, 32:160], atol=0, rtol=0)


def test_model_config_from_hf_dir(tmp_path):
    path = _save(_hf("qwen3_next"), tmp_path)
    cfg = ModelConfig.from_pretrained(path)
    assert cfg.model_type == "qwen3_next" and cfg.layer_kind(0) == "gdn" and cfg.layer_kind(1) == "attention"
    assert cfg.num_experts == 8 and cfg.shared_expert_intermediate_size == 128 and cfg.attn_output_gate


def test_fast_loader_gives_identical_tensors(tmp_path, monkeypatch):
    path = _save(_hf("qwen3"), tmp_path)
    slow = Checkpoint(path)
    monkeypatch.setenv("ATLAS_FAST_LOAD", "1")
    fast = Checkpoint(path)
    assert fast._fast and set(fast.keys()) == set(slow.keys())
    for k in slow.keys():
        a, b = slow.get(k), fast.get(k)
        assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
    m = load_model(path, dtype="float32", with_mtp=False)
    assert m.layers[0].mixer.qkv.weight.shape[1] == 256


def test_multimodal_logits_match_transformers(tmp_path):
    """Qwen3.5 with its vision tower: an image in the middle of the prompt.  The tower output, the placeholder
    substitution and the interleaved three-stream rotary positions together must reproduce the HF logits; a chunked
    prefill followed by decode steps through the engine must continue at the right positions after the image."""
    from atlas_b200.config import EngineConfig
    from atlas_b200.engine import LLMEngine
    from atlas_b200.models.batch import ForwardBatch
    from atlas_b200.models.vision import prepare
    from atlas_b200.sampling import SamplingParams
    torch.manual_seed(0)
    tc = dict(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
              max_position_embeddings=256, intermediate_size=512, linear_num_key_heads=2, linear_num_value_heads=4,
              linear_key_head_dim=64, linear_value_head_dim=64, layer_types=["linear_attention", "full_attention"],
              tie_word_embeddings=False)
    vc = dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4, temporal_patch_size=2,
              spatial_merge_size=2, out_hidden_size=256, num_position_embeddings=64)
    cfg = transformers.Qwen3_5Config(text_config=tc, vision_config=vc, image_token_id=500, video_token_id=501,
                                     vision_start_token_id=502, vision_end_token_id=503)
    hf = transformers.Qwen3_5ForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias") or "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    path = _save(hf, tmp_path)
    grid = (1, 4, 6)                                            # 24 patches -> 6 placeholders
    px = torch.randn(24, 3 * 2 * 4 * 4)
    toks = [11, 12, 502] + [500] * 6 + [503, 13, 14, 15, 16, 17]
    types = [1 if t == 500 else 0 for t in toks]
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([toks]), pixel_values=px, image_grid_thw=torch.tensor([grid]),
                  mm_token_type_ids=torch.tensor([types])).logits[0]
    model = load_model(path, dtype="float32", with_mtp=False)
    assert model.vision is not None and model.cfg.image_token_id == 500
    mm = prepare(model.vision, toks, 500, [(px, grid)])
    assert mm.delta == 3 - 6                                    # the image advances positions by max(2, 3), not by 6 tokens
    cache = model.alloc_cache(4, 16, torch.float32, state_slots=1)
    fb = ForwardBatch.build([toks], [0], [[0, 1, 2]], 16, state_slots=[0], has_state=[False], all_logits=True)
    fb.positions3 = torch.from_numpy(mm.positions(0, len(toks)))
    emb = model.embed_tokens(fb.input_ids).clone()
    emb[torch.tensor(types).bool()] = mm.embeds
    fb.inputs_embeds = emb
    got = model.compute_logits(model.forward(fb, cache))
    torch.testing.assert_close(got, want, atol=3e-4, rtol=1e-3)
    # through the engine: chunked prefill (8-token chunks cut the image in two), then greedy decode; the oracle decodes
    # by re-running the whole sequence
    eng = LLMEngine(model, EngineConfig(num_kv_blocks=16, max_num_seqs=2, max_seq_len=64, max_prefill_tokens=8,
                                        enable_prefix_caching=False))
    eng.add_request(toks, SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True), images=[(px, grid)])
    out = []
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                out = o.output_tokens
    seq = list(toks)
    ref_out = []
    for _ in range(4):
        with torch.no_grad():
            lg = hf(input_ids=torch.tensor([seq]), pixel_values=px, image_grid_thw=torch.tensor([grid]),
                    mm_token_type_ids=torch.tensor([[1 if t == 500 else 0 for t in seq]])).logits[0, -1]
        nxt = int(lg.argmax())
        ref_out.append(nxt)
        seq.append(nxt)
    assert out == ref_out


@pytest.mark.parametrize("fmt", ["mxfp4", "mlx4", "mlx8"])
def test_other_weight_containers(fmt, tmp_path):
    """MXFP4 (32-value e2m1 blocks + e8m0 scales) and MLX affine group quantisation: a checkpoint rewritten in the
    container loads and reproduces the logits of the same weights dequantised by hand."""
    from safetensors.torch import load_file, save_file
    hf = _hf("llama")
    src = _save(hf, tmp_path / "src")
    tensors = load_file(os.path.join(src, "model.safetensors"))
    out, deq = {}, {}
    for name, t in tensors.items():
        if not (name.endswith("_proj.weight") and t.dim() == 2):
            out[name] = deq[name] = t
            continue
        base = name[:-len(".weight")]
        if fmt == "mxfp4":
            b, sc = Q.quantize_mxfp4(t.float())
            out[base + ".weight_blocks"], out[base + ".weight_scales"] = b, sc
            deq[name] = Q.dequantize_mxfp4(b, sc)
        else:
            bits = 4 if fmt == "mlx4" else 8
            w, sc, bi = Q.quantize_mlx(t.float(), bits, 64)
            out[name], out[base + ".scales"], out[base + ".biases"] = w, sc, bi
            deq[name] = Q.dequantize_mlx(w, sc, bi, bits, 64)
            assert float((deq[name] - t.float()).abs().max()) < (0.02 if bits == 4 else 0.002)
    dst = tmp_path / fmt
    os.makedirs(dst)
    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(dst, "model.safetensors"))
    cfg = json.load(open(os.path.join(src, "config.json")))
    if fmt == "mxfp4":
        cfg["quantization_config"] = {"quant_method": "mxfp4"}
    else:
        cfg["quantization"] = {"group_size": 64, "bits": 4 if fmt == "mlx4" else 8}
    json.dump(cfg, open(os.path.join(dst, "config.json"), "w"))
    model = load_model(str(dst), dtype="float32", with_mtp=False)
    if fmt == "mxfp4":
        assert model.layers[0].mixer.qkv.kind == "nvfp4"            # kept in 4 bits, on the NVFP4 kernels' layout
    toks = torch.randint(0, 512, (20,), generator=torch.Generator().manual_seed(7)).tolist()
    got = _ours_logits(model, toks)
    hf.load_state_dict({k: v.to(torch.float32) for k, v in deq.items()})
    with torch.no_grad():
        want = hf(torch.tensor([toks])).logits[0]
    torch.testing.assert_close(got, want, atol=2e-3 if fmt == "mlx4" else 5e-4, rtol=1e-3)
