"""LoRA adapters: per-request application must equal a model whose weights had the low-rank update merged in, requests
with and without an adapter can share a batch, and the PEFT directory layout loads."""
import json
import os

import torch
from safetensors.torch import save_file

from atlas_b200.config import EngineConfig, tiny_dense
from atlas_b200.engine import LLMEngine
from atlas_b200.lora import load_adapter
from atlas_b200.models import build_model
from atlas_b200.sampling import SamplingParams

MODS = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj",
        "mlp.down_proj"]


def _write_adapter(path, cfg, r=4, seed=0):
    g = torch.Generator().manual_seed(seed)
    h, kv, i = cfg.hidden_size, cfg.kv_size, cfg.intermediate_size
    dims = {"self_attn.q_proj": (cfg.q_size, h), "self_attn.k_proj": (kv, h), "self_attn.v_proj": (kv, h),
            "self_attn.o_proj": (h, cfg.q_size), "mlp.gate_proj": (i, h), "mlp.up_proj": (i, h), "mlp.down_proj": (h, i)}
    tensors = {}
    for layer in range(cfg.num_hidden_layers):
        for m in MODS:
            out, inp = dims[m]
            tensors[f"base_model.model.model.layers.{layer}.{m}.lora_A.weight"] = torch.randn(r, inp, generator=g) * 0.05
            tensors[f"base_model.model.model.layers.{layer}.{m}.lora_B.weight"] = torch.randn(out, r, generator=g) * 0.05
    os.makedirs(path, exist_ok=True)
    save_file(tensors, os.path.join(path, "adapter_model.safetensors"))
    json.dump({"r": r, "lora_alpha": 8, "target_modules": [m.split(".")[-1] for m in MODS]}, open(os.path.join(path, "adapter_config.json"), "w"))
    return path


def _merged(model, adapter):
    """A second model whose dense weights carry W + scaling * B A."""
    cfg = model.cfg
    m2 = build_model(cfg).init_random(0)
    nq, nkv = cfg.q_size, cfg.kv_size
    for l, (a, b) in enumerate(zip(model.layers, m2.layers)):
        d = lambda name: adapter.scaling * (adapter.weights[f"layers.{l}.{name}"][1].float() @ adapter.weights[f"layers.{l}.{name}"][0].float())
        w = b.mixer.qkv.weight
        w[:nq] += d("self_attn.q_proj"); w[nq:nq + nkv] += d("self_attn.k_proj"); w[nq + nkv:nq + 2 * nkv] += d("self_attn.v_proj")
        b.mixer.o.weight += d("self_attn.o_proj")
        i = cfg.intermediate_size
        b.ffn.gate_up.weight[:i] += d("mlp.gate_proj"); b.ffn.gate_up.weight[i:] += d("mlp.up_proj")
        b.ffn.down.weight += d("mlp.down_proj")
    return m2


def test_lora_equals_merged_weights_and_mixes_in_a_batch(tmp_path):
    cfg = tiny_dense()
    model = build_model(cfg).init_random(0)
    adapter = load_adapter(_write_adapter(str(tmp_path / "ad1"), cfg), model)
    assert adapter.rank == 4 and len(adapter.weights) == cfg.num_hidden_layers * len(MODS)
    slot = model.enable_lora().register(adapter)
    assert slot == 1 and model.lora.slot_of("ad1") == 1 and model.lora.slot_of(None) == 0
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (20,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    ecfg = EngineConfig(num_kv_blocks=64, max_num_seqs=8, enable_prefix_caching=False)
    base = [o.output_tokens for o in LLMEngine(build_model(cfg).init_random(0), ecfg).generate(prompts, sp)]
    merged = [o.output_tokens for o in LLMEngine(_merged(model, adapter), ecfg).generate(prompts, sp)]
    assert base != merged                                    # the adapter changes the output at all
    eng = LLMEngine(model, ecfg)
    ids = [eng.add_request(prompts[0], SamplingParams(max_tokens=8, ignore_eos=True), adapter_slot=1),
           eng.add_request(prompts[1], SamplingParams(max_tokens=8, ignore_eos=True)),
           eng.add_request(prompts[2], SamplingParams(max_tokens=8, ignore_eos=True), adapter_slot=1)]
    done = {}
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                done[o.request_id] = list(o.output_tokens)
    assert done[ids[0]] == merged[0] and done[ids[2]] == merged[2]      # adapter rows
    assert done[ids[1]] == base[1]                                      # base-model row in the same batch
