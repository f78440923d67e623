#!/usr/bin/env python
"""Headline benchmark: aggregate output tokens/s of a wave of concurrent requests (the reference's
concurrency-sweep metric) on a Llama-3-8B-shaped FP8 block-scaled decoder with an FP8 KV cache.

One *step* is one full wave: ``--concurrency`` requests of ``--isl`` random input tokens each generate
``--osl`` tokens (EOS ignored) through ``LLMEngine`` (continuous batching, chunked prefill, paged KV).
``--gpus N`` runs tensor-parallel over N GPUs (launch with torchrun for N > 1).

Prints one JSON line.  ``value`` is output tokens / CUDA-event time of the steps' GPU work;
``e2e.value`` is output tokens / wall time of the same waves through the public API, including every step's
pinned-host -> device input copies and the device -> host read of the sampled tokens.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_TOK_S = None   # the reference publishes no number for this config on any hardware


def _clock_sampler(gpu_index: int):
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        return subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200",
                                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except Exception:
        return None


def _clock_summary(proc):
    if proc is None:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    proc.terminate()
    try:
        out, _ = proc.communicate(timeout=5)
    except Exception:
        proc.kill()
        out = ""
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in out.splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 9:
            continue
        try:
            sm.append(float(f[1]))
            mx.append(float(f[2]))
        except ValueError:
            continue
        for n, v in zip(names, f[5:9]):
            if v.lower().startswith("active"):
                reasons.add(n)
    if not sm:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
    busy = sorted(sm)[len(sm) // 4:]       # drop the idle tail of samples
    return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def _torch_nccl_arm(args, mcfg, topo, device, real_stdout) -> int:
    """This repository's own library baseline (see ``atlas_b200/bench/torch_baseline.py``): same wave, same model shape,
    stock PyTorch / cuBLASLt / NCCL kernels only."""
    import torch
    from atlas_b200.bench.torch_baseline import TorchNcclDecoder
    world, rank = topo.world_size, topo.rank
    model = TorchNcclDecoder(mcfg, rank, world, device)
    model.alloc_cache(args.concurrency, args.isl + args.osl + 8)
    gen = torch.Generator().manual_seed(1234)
    pinned = torch.empty(args.concurrency, args.isl, dtype=torch.long).pin_memory()

    def wave():
        pinned.copy_(torch.randint(0, mcfg.vocab_size, (args.concurrency, args.isl), generator=gen))
        return model.wave(pinned, args.osl)

    def sync_all():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
    for _ in range(max(1, min(args.warmup, 3))):
        wave()
    sync_all()
    sampler = _clock_sampler(torch.cuda.current_device()) if rank == 0 else None
    t0 = time.perf_counter()
    tokens, dev_s, ttfts = 0, 0.0, []
    for _ in range(args.steps):
        n, tt, d = wave()
        tokens += n
        dev_s += d
        ttfts += tt
    sync_all()
    wall = time.perf_counter() - t0
    clocks = _clock_summary(sampler) if rank == 0 else None
    t = torch.tensor([wall, dev_s], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    wall, dev_s = float(t[0]), float(t[1])
    if rank == 0:
        line = {"metric": "aggregate output tok/s (concurrency wave, ISL/OSL)", "value": round(tokens / dev_s, 2), "unit": "tok/s",
                "n_gpus": world, "steps": args.steps, "warmup": min(args.warmup, 3), "ms_per_step": round(wall * 1e3 / args.steps, 3),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "fp8-e4m3 weights and activations (row-wise scales, cuBLASLt), bf16 KV",
                "data": "synthetic: uniform-random token ids, random-init N(0,0.02) weights quantized to fp8",
                "config": {"model": args.model, "global_batch": args.concurrency, "seq_len": args.isl + args.osl, "isl": args.isl,
                           "osl": args.osl, "parallelism": f"tp{topo.tp_size}" + (f"+ep{topo.ep_size}" if topo.ep_size > 1 else ""), "collectives": "nccl" if world > 1 else "none",
                           "l2": "inputs larger than L2", "step": "one wave of `global_batch` concurrent requests, prefill + decode",
                           "note": "THIS REPOSITORY'S OWN BASELINE, not the upstream reference: eager PyTorch, torch._scaled_mm, "
                                   "SDPA, dense KV cache, static batch, no scheduler, no CUDA graphs"},
                "clocks": clocks,
                "e2e": {"value": round(tokens / wall, 2), "unit": "tok/s", "h2d_bytes_per_step": args.concurrency * args.isl * 8,
                        "d2h_bytes_per_step": args.concurrency * args.osl * 8, "note": "per wave"},
                "gpu_launches": 0, "ttft_p50_ms": round(statistics.median(ttfts) * 1e3, 2),
                "tpot_ms": round((wall / args.steps) * 1e3 / args.osl, 3), "impl": "torch-nccl (own baseline)"}
        os.write(real_stdout, (json.dumps(line) + "\n").encode())
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="atlas_b200", choices=["atlas_b200", "reference", "torch-nccl"],
                    help="atlas_b200: this engine; reference: the upstream project (not buildable here, prints why); "
                         "torch-nccl: this repository's own library baseline (torch._scaled_mm + SDPA + NCCL, eager)")
    ap.add_argument("--ladder", default="1,8,32", help="extra concurrency rungs reported under `ladder` ('' = none)")
    ap.add_argument("--ladder-steps", type=int, default=2)
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--concurrency", type=int, default=128)
    ap.add_argument("--isl", type=int, default=1024)
    ap.add_argument("--osl", type=int, default=256)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-prefill-tokens", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (marks the result invalid)")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--speculative", action="store_true", help="MTP speculative decoding (models with a draft head)")
    ap.add_argument("--num-drafts", type=int, default=3)
    ap.add_argument("--prefix-cache", action="store_true")
    ap.add_argument("--shared-prefix", type=int, default=0, help="every second prompt starts with the same N tokens")
    ap.add_argument("--ep", type=int, default=0,
                    help="expert-parallel size for MoE models (0 = none; N = every rank owns 1/N of the experts while attention "
                         "stays tensor parallel over all ranks)")
    ap.add_argument("--ep-mode", default="auto", choices=["auto", "allreduce", "alltoall"],
                    help="expert-parallel data path: local experts + fused combine/all-reduce, or peer-memory all-to-all")
    ap.add_argument("--ngram-speculative", action="store_true", help="prompt-lookup drafts (no draft model), --num-drafts deep")
    ap.add_argument("--kv-cache-dtype", default="fp8", choices=["fp8", "bf16", "nvfp4", "turbo8"], help="paged KV cache dtype (the headline uses fp8)")
    ap.add_argument("--self-speculative", action="store_true", help="layer-skipping drafts from the target model itself")
    ap.add_argument("--nvfp4-activations", action="store_true",
                    help="NVFP4 checkpoints: quantise activations to NVFP4 too (block-scaled FP4 x FP4 tensor-core GEMM)")
    ap.add_argument("--ssm-checkpoint-interval", type=int, default=0,
                    help="hybrid models: tokens between recurrent-state snapshots for the prefix cache (0 = engine default)")
    ap.add_argument("--ssm-cache-slots", type=int, default=0, help="hybrid models: snapshot slots (0 = concurrency + 8)")
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"],
                    help="tensor-parallel collectives: this engine's peer-memory kernels (default) or the NCCL baseline")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "refused by a safety check: pip install of the reference checkout was denied; the reference is a Rust "
                          "workspace (no setup.py/pyproject.toml, needs cargo which the image lacks)"}))
        return 0

    # Libraries (NCCL's version banner among them) print to file descriptor 1 on their own; the contract is ONE JSON
    # line on stdout, so everything else is sent to stderr and the result line is written to the saved descriptor.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    import torch
    from atlas_b200.config import PRESETS, EngineConfig
    from atlas_b200.engine import LLMEngine
    from atlas_b200.models import build_model
    from atlas_b200.parallel import init_distributed
    from atlas_b200.sampling import SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if args.gpus > 1:
            print(f"bench.py: --gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})", file=sys.stderr)
            return 2
    topo, pctx, device = init_distributed(tp_size=world, ep_size=args.ep if world > 1 else 0, timeout_s=180.0)
    rank = topo.rank
    if args.nvfp4_activations:
        from atlas_b200 import ops as _ops
        _ops.NVFP4_ACTIVATIONS = True
    from atlas_b200.ops import cuda as K
    symm = None
    if world > 1 and args.comm == "p2p":
        from atlas_b200.parallel.symm import SymmBackend
        symm = SymmBackend(pctx.comm, device)
        if pctx.ep_comm is pctx.comm:
            pctx.ep_comm = symm
        pctx.comm = symm

    mcfg = PRESETS[args.model]()
    if args.layers:
        mcfg.num_hidden_layers = args.layers
    if args.impl == "torch-nccl":
        rc = _torch_nccl_arm(args, mcfg, topo, device, real_stdout)
        if world > 1:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()
        return rc
    max_len = args.isl + args.osl + 16
    mcfg.max_position_embeddings = max(4096, max_len)
    model = build_model(mcfg, pctx, device=device, ep_mode=args.ep_mode).init_random(0, max_pos=max_len + 16)
    blocks_per_seq = (max_len + args.block_size - 1) // args.block_size + 1
    ecfg = EngineConfig(max_seq_len=max_len, block_size=args.block_size, max_num_seqs=max(args.concurrency, 1),
                        max_batch_size=max(args.concurrency, 1), max_prefill_tokens=args.max_prefill_tokens,
                        num_kv_blocks=blocks_per_seq * args.concurrency + 64, enable_prefix_caching=args.prefix_cache,
                        speculative=args.speculative, ngram_speculative=args.ngram_speculative, self_speculative=args.self_speculative,
                        num_drafts=args.num_drafts if (args.speculative or args.ngram_speculative or args.self_speculative) else 0,
                        ssm_cache_slots=args.ssm_cache_slots or max(16, args.concurrency + 8),
                        **({"ssm_checkpoint_interval": args.ssm_checkpoint_interval} if args.ssm_checkpoint_interval else {}),
                        use_cuda_graphs=not args.no_graphs, tp_size=world, kv_cache_dtype=args.kv_cache_dtype)
    eng = LLMEngine(model, ecfg)
    eng.time_device = True
    sp = SamplingParams(max_tokens=args.osl, temperature=0.0, ignore_eos=True)
    gen = torch.Generator().manual_seed(1234)

    def wave(conc=None):
        conc = conc or args.concurrency
        prompts = [torch.randint(0, mcfg.vocab_size, (args.isl,), generator=gen).tolist() for _ in range(conc)]
        if args.shared_prefix:
            shared = torch.randint(0, mcfg.vocab_size, (args.shared_prefix,), generator=gen).tolist()
            for i in range(0, len(prompts), 2):
                prompts[i][:args.shared_prefix] = shared
        outs = eng.generate(prompts, sp)
        return sum(len(o.output_tokens) for o in outs), [o.ttft_s for o in outs]

    def sync_all():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        wave()
    sync_all()
    st = K.check_status()
    if st:
        print(f"bench.py: device status word {st:#x} after warm-up", file=sys.stderr)
        return 3
    sampler = _clock_sampler(torch.cuda.current_device()) if rank == 0 else None
    eng.device_time_ms = 0.0
    eng.device_phase_ms = {}
    launches0, replays0 = K.launch_count, eng.runner.graph_replays
    h2d0 = eng.runner.h2d_bytes
    steps0 = eng.stats.steps
    sync_all()
    t0 = time.perf_counter()
    tokens = 0
    ttfts = []
    for _ in range(args.steps):
        n, tt = wave()
        tokens += n
        ttfts += [t for t in tt if t is not None]
    sync_all()
    wall = time.perf_counter() - t0
    clocks = _clock_summary(sampler) if rank == 0 else None
    dev_s = eng.device_time_ms / 1e3
    st = K.check_status()
    if st:
        # a bounded device-side wait gave up inside the timed region: whatever was timed is not the workload
        print(f"bench.py: device status word {st:#x} after the timed waves: result discarded", file=sys.stderr)
        return 3
    main_launches = (K.launch_count - launches0) + (eng.runner.graph_replays - replays0) * eng.runner.kernels_per_graph()
    main_steps, main_h2d = eng.stats.steps - steps0, eng.runner.h2d_bytes - h2d0
    main_phase = {k: {"ms": round(v[0], 1), "engine_steps": v[1]} for k, v in eng.device_phase_ms.items()}
    # the lower rungs of the concurrency ladder (same engine, same request shape): one warm-up wave, then timed waves
    ladder = []
    for c in [int(x) for x in args.ladder.split(",") if x.strip()]:
        if c >= args.concurrency:
            continue
        wave(c)
        sync_all()
        eng.device_time_ms = 0.0
        w0 = time.perf_counter()
        n_tok, tt_all = 0, []
        for _ in range(max(1, args.ladder_steps)):
            n, tt = wave(c)
            n_tok += n
            tt_all += [t for t in tt if t is not None]
        sync_all()
        w = time.perf_counter() - w0
        tl = torch.tensor([w, eng.device_time_ms / 1e3], dtype=torch.float64, device=device)
        if world > 1:
            torch.distributed.all_reduce(tl, op=torch.distributed.ReduceOp.MAX)
        w, d_s = float(tl[0]), float(tl[1])
        ladder.append({"concurrency": c, "value": round(n_tok / d_s, 2) if d_s > 0 else None, "e2e": round(n_tok / w, 2),
                       "ttft_p50_ms": round(statistics.median(tt_all) * 1e3, 2) if tt_all else None,
                       "tpot_ms": round(w / max(1, args.ladder_steps) * 1e3 / args.osl, 3)})
    if K.check_status():
        print("bench.py: device status word set during the ladder rungs", file=sys.stderr)
        return 3
    t = torch.tensor([wall, dev_s], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    wall, dev_s = float(t[0]), float(t[1])
    eng_steps, launches = main_steps, main_launches
    qm = mcfg.quant.method
    dtype_desc = {"fp8_block": "fp8-e4m3 weights (128x128 scales) + fp8 KV, bf16 activations",
                  "nvfp4": "nvfp4 weights (e2m1, e4m3 scale per 16, fp32 global)" + (" for experts, bf16 elsewhere" if mcfg.quant.experts_only else "") + " + fp8 KV, bf16 activations",
                  }.get(qm, "bf16 weights + fp8 KV")
    if args.kv_cache_dtype != "fp8":
        dtype_desc = dtype_desc.replace("fp8 KV", f"{args.kv_cache_dtype} KV")
    quant_desc = {"fp8_block": " quantized to fp8 block-scaled", "nvfp4": " quantized to nvfp4"}.get(qm, "")
    if rank == 0:
        value = tokens / dev_s if dev_s > 0 else 0.0
        e2e = tokens / wall
        line = {
            "metric": "aggregate output tok/s (concurrency wave, ISL/OSL)", "value": round(value, 2), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(wall * 1e3 / args.steps, 3), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / BASELINE_TOK_S) if BASELINE_TOK_S else None, "dtype": dtype_desc,
            "data": "synthetic: uniform-random token ids, random-init N(0,0.02) weights" + quant_desc,
            "config": {"model": args.model + ("" if not args.layers else f"-TRUNCATED-{args.layers}L-INVALID"),
                       "global_batch": args.concurrency, "seq_len": args.isl + args.osl, "isl": args.isl, "osl": args.osl,
                       "parallelism": f"tp{topo.tp_size}" + (f"+ep{topo.ep_size}" if topo.ep_size > 1 else ""), "collectives": (args.comm if world > 1 else "none"), "l2": "inputs larger than L2 (8 GB weights + KV stream every step)",
                       "step": "one wave of `global_batch` concurrent requests, prefill + decode",
                       "engine_steps_per_wave": eng_steps / max(1, args.steps), "cuda_graphs": not args.no_graphs,
                       "speculative": bool(args.speculative or args.ngram_speculative or args.self_speculative), "nvfp4_activations": bool(args.nvfp4_activations),
                       "ep_mode": args.ep_mode if topo.ep_size > 1 else None, "prefix_cache": bool(args.prefix_cache),
                       "spec_accept_rate": (eng.stats.spec_accepted / eng.stats.spec_proposed) if eng.stats.spec_proposed else None,
                       "prefix_hit_tokens": (eng.radix.stats.hit_tokens if eng.radix is not None else 0)},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 2), "unit": "tok/s",
                    "h2d_bytes_per_step": int(main_h2d / max(1, eng_steps)),
                    "d2h_bytes_per_step": int(8 * tokens / max(1, eng_steps)),
                    "note": "per engine step; every step copies token ids / positions / slots / block tables from pinned host memory and reads the sampled token ids back"},
            "gpu_launches": int(launches),
            "ttft_p50_ms": round(statistics.median(ttfts) * 1e3, 2) if ttfts else None,
            "tpot_ms": round((wall / args.steps) * 1e3 / args.osl, 3),
            "device_phase_ms": main_phase,
            "ladder": ladder,
            "impl": "atlas_b200",
        }
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        torch.distributed.barrier()
        if symm is not None:
            symm.close()
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
