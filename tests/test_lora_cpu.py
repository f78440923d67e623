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


def _run_requests(eng, prompts, slots):
    ids = [eng.add_request(p, SamplingParams(max_tokens=8, ignore_eos=True), adapter_slot=s) for p, s in zip(prompts, slots)]
    done = {}
    while len(done) < len(ids):
        for o in eng.step():
            if o.finished:
                done[o.request_id] = list(o.output_tokens)
    return [done[i] for i in ids]


def test_lora_on_tensor_parallel_ranks_equals_one_process(tmp_path):
    """Each rank reads the adapter itself, keeps the slices that match its shard of the base weights, and adds the
    row-parallel partial deltas before the group reduction: tokens equal the unsharded engine's, adapter rows and base
    rows mixed.  The adapter reaches the followers as a control-plane event ahead of the requests that name its slot."""
    from atlas_b200.layers.common import ParallelCtx
    from atlas_b200.parallel.comm import FakeWorld
    from atlas_b200.parallel.worker import DistributedEngine, StepControl, worker_loop
    cfg = tiny_dense()
    path = _write_adapter(str(tmp_path / "ad1"), cfg)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (20,), generator=g).tolist() for _ in range(3)]
    ecfg = EngineConfig(num_kv_blocks=64, max_num_seqs=8, enable_prefix_caching=False)
    one = LLMEngine(build_model(cfg).init_random(0), ecfg)
    assert one.load_adapter("ad1", path) == 1
    want = _run_requests(one, prompts, [1, 0, 1])

    data, ctrl = FakeWorld(2, timeout_s=20.0), FakeWorld(2, timeout_s=20.0)
    followers = [None, None]

    def rank_fn(r):
        comm = data.comm(r)
        pctx = ParallelCtx(tp_rank=r, tp_size=2, ep_rank=r, ep_size=2, comm=comm, ep_comm=comm)
        eng = LLMEngine(build_model(cfg, pctx).init_random(0), ecfg)
        control = StepControl(ctrl.comm(r), heartbeat_s=0.05)
        if r == 0:
            de = DistributedEngine(eng, control)
            try:
                assert de.load_adapter("ad1", path) == 1
                return _run_requests(de, prompts, [1, 0, 1])
            finally:
                de.shutdown()
        followers[r] = eng
        return worker_loop(eng, control)

    got = data.run(rank_fn, timeout_s=120.0)[0]
    assert got == want
    ad = followers[1].model.lora.slots[1]
    assert ad.weights["layers.0.self_attn.o_proj"][0].shape[1] == cfg.q_size // 2        # A cut along the input
    assert ad.weights["layers.0.mlp.gate_proj"][1].shape[0] == cfg.intermediate_size // 2  # B cut along the output


def _write_moe_adapter(path, cfg, r=4, seed=1, experts=(0, 3, 5)):
    g = torch.Generator().manual_seed(seed)
    h, i = cfg.hidden_size, cfg.moe_intermediate_size
    t = {}
    for layer in range(cfg.num_hidden_layers):
        pre = f"base_model.model.model.layers.{layer}.mlp."
        t[pre + "gate.lora_A.weight"] = torch.randn(r, h, generator=g) * 0.05
        t[pre + "gate.lora_B.weight"] = torch.randn(cfg.num_experts, r, generator=g) * 0.05
        for e in experts:
            for leaf, (out, inp) in {"gate_proj": (i, h), "up_proj": (i, h), "down_proj": (h, i)}.items():
                t[f"{pre}experts.{e}.{leaf}.lora_A.weight"] = torch.randn(r, inp, generator=g) * 0.08
                t[f"{pre}experts.{e}.{leaf}.lora_B.weight"] = torch.randn(out, r, generator=g) * 0.08
    os.makedirs(path, exist_ok=True)
    save_file(t, os.path.join(path, "adapter_model.safetensors"))
    json.dump({"r": r, "lora_alpha": 8}, open(os.path.join(path, "adapter_config.json"), "w"))
    return path


def _merged_moe(cfg, adapter):
    from atlas_b200.config import tiny_moe  # noqa: F401  (the caller's cfg)
    m2 = build_model(cfg).init_random(0)
    i = cfg.moe_intermediate_size
    for l, layer in enumerate(m2.layers):
        d = lambda name: adapter.scaling * (adapter.weights[name][1].float() @ adapter.weights[name][0].float())
        pre = f"layers.{l}.mlp."
        layer.ffn.router.weight += d(pre + "gate")
        for e in range(cfg.num_experts):
            if pre + f"experts.{e}.gate_proj" in adapter.weights:
                layer.ffn.experts.w13[e, :i] += d(pre + f"experts.{e}.gate_proj")
                layer.ffn.experts.w13[e, i:] += d(pre + f"experts.{e}.up_proj")
                layer.ffn.experts.w2[e] += d(pre + f"experts.{e}.down_proj")
    return m2


def test_moe_router_and_expert_lora_equal_merged_weights(tmp_path):
    from atlas_b200.config import tiny_moe
    cfg = tiny_moe()
    model = build_model(cfg).init_random(0)
    eng = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=8, enable_prefix_caching=False))
    assert eng.load_adapter("moe-ad", _write_moe_adapter(str(tmp_path / "moe"), cfg)) == 1
    adapter = load_adapter(str(tmp_path / "moe"))
    assert model.lora.slots[1].expert_layers() == set(range(cfg.num_hidden_layers))
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 1024, (20,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    ecfg = EngineConfig(num_kv_blocks=64, max_num_seqs=8, enable_prefix_caching=False)
    base = [o.output_tokens for o in LLMEngine(build_model(cfg).init_random(0), ecfg).generate(prompts, sp)]
    merged = [o.output_tokens for o in LLMEngine(_merged_moe(cfg, adapter), ecfg).generate(prompts, sp)]
    assert base != merged
    got = _run_requests(eng, prompts, [1, 0, 1])
    assert got[0] == merged[0] and got[2] == merged[2] and got[1] == base[1]


def test_moe_expert_lora_on_expert_parallel_ranks(tmp_path):
    """Two expert-parallel ranks: each recomputes the adapter rows over its own experts and the group sums them."""
    from atlas_b200.config import tiny_moe
    from atlas_b200.layers.common import ParallelCtx
    from atlas_b200.parallel.comm import FakeWorld
    cfg = tiny_moe()
    path = _write_moe_adapter(str(tmp_path / "moe"), cfg)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 1024, (20,), generator=g).tolist() for _ in range(3)]
    ecfg = EngineConfig(num_kv_blocks=64, max_num_seqs=8, enable_prefix_caching=False)
    one = LLMEngine(build_model(cfg).init_random(0), ecfg)
    one.load_adapter("moe-ad", path)
    want = _run_requests(one, prompts, [1, 0, 1])
    world = FakeWorld(2, timeout_s=20.0)

    def rank_fn(r):
        comm = world.comm(r)
        pctx = ParallelCtx(tp_rank=r, tp_size=2, ep_rank=r, ep_size=2, comm=comm, ep_comm=comm)
        eng = LLMEngine(build_model(cfg, pctx).init_random(0), ecfg)
        eng.load_adapter("moe-ad", path)
        return _run_requests(eng, prompts, [1, 0, 1])

    outs = world.run(rank_fn, timeout_s=120.0)
    assert outs[0] == want and outs[1] == want
