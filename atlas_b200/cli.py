"""Command line: ``python -m atlas_b200 {serve,benchmark,doctor,recipes}``.

``serve`` boots in phases: arguments (+ recipe) -> rank topology / process group -> model (checkpoint directory or a
``preset:<name>`` random-init shape) -> engine (KV sizing, CUDA graphs) -> on rank 0 the HTTP server and scheduler
thread, on the other ranks the follower loop.  One OS process per GPU; start N ranks with ``torchrun`` or pass
``--rank/--world-size/--master-addr/--master-port`` to each process.

Reference parity: ``crates/spark-server/src/cli/serve_args.rs`` (flag names and defaults),
``main_modules/serve.rs:58`` + ``serve_phases/*`` (boot phases), ``main_modules/serve_phases/build.rs:211-330``
(rank 0 serves, ranks > 0 run the worker step loop).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="atlas_b200", description="Blackwell-native LLM inference engine")
    sub = ap.add_subparsers(dest="cmd", required=True)

    s = sub.add_parser("serve", help="serve a model over HTTP (OpenAI / Anthropic / Responses APIs)")
    s.add_argument("model", nargs="?", help="checkpoint directory, or preset:<name> for a random-init shape")
    s.add_argument("--recipe", help="recipe id or YAML path; its defaults apply below explicit flags")
    s.add_argument("--served-model-name")
    s.add_argument("--port", type=int, default=8888)
    s.add_argument("--bind", default="0.0.0.0")
    s.add_argument("--max-seq-len", type=int, default=32768)
    s.add_argument("--block-size", type=int, default=16)
    s.add_argument("--no-logit-pipeline", action="store_true",
                   help="do not attach the think / tool-call logit stages (mid-word close defer, post-close masks, tool-call pin)")
    s.add_argument("--margin-counter", action="store_true",
                   help="count decode positions with a small top-1 / top-2 gap (one device read-back per token of the requests it covers)")
    s.add_argument("--think-confidence-streak", type=int, default=0,
                   help="end thinking early after this many consecutive tokens with top-1 probability >= 0.95 (0 = off)")
    s.add_argument("--mtp-vocab", type=int, default=0, help="draft steps score this many rows of the lm_head (0 = all)")
    s.add_argument("--mtp-vocab-rank", default="id", help="'id' (first rows) or the path of a ranked token-id table")
    s.add_argument("--kv-cache-dtype", default="fp8", choices=["auto", "fp8", "bf16", "nvfp4", "turbo8"])
    s.add_argument("--sparse-attention-blocks", type=int, default=0,
                   help="long contexts: decode attention reads at most this many KV blocks per sequence, chosen by a "
                        "block predictor (first and most recent blocks always kept); 0 = dense attention")
    s.add_argument("--dcut-ratio", type=float, default=0.0,
                   help="speculative decoding: verify only this fraction of the draft rows (0.25 / 0.5 / 0.75), chosen by drafter confidence")
    s.add_argument("--kv-high-precision-layers", default="",
                   help="comma-separated attention layer indices that keep a bf16 KV cache when the rest is FP8")
    s.add_argument("--gpu-memory-utilization", type=float, default=0.90)
    s.add_argument("--num-kv-blocks", type=int, default=None)
    s.add_argument("--max-num-seqs", type=int, default=128)
    s.add_argument("--max-batch-size", type=int, default=128)
    s.add_argument("--max-prefill-tokens", type=int, default=8192)
    s.add_argument("--scheduling-policy", default="fifo", choices=["fifo", "slai"])
    s.add_argument("--tbt-deadline-ms", type=float, default=100.0)
    s.add_argument("--enable-prefix-caching", action="store_true", default=None)
    s.add_argument("--no-prefix-caching", dest="enable_prefix_caching", action="store_false")
    s.add_argument("--speculative", action="store_true")
    s.add_argument("--num-drafts", type=int, default=0)
    s.add_argument("--ngram-speculative", action="store_true", help="prompt-lookup drafts (no draft model)")
    s.add_argument("--self-speculative", action="store_true", help="layer-skipping drafts from the target model itself")
    s.add_argument("--self-spec-keep", type=float, default=0.5, help="fraction of the layers a self-speculative draft pass runs")
    s.add_argument("--ngram-max", type=int, default=4)
    s.add_argument("--ngram-min", type=int, default=2)
    s.add_argument("--mtp-gate", action="store_true", default=None)
    s.add_argument("--no-mtp-gate", dest="mtp_gate", action="store_false")
    s.add_argument("--ssm-cache-slots", type=int, default=16)
    s.add_argument("--ssm-checkpoint-interval", type=int, default=256)
    s.add_argument("--swap-space-gb", type=float, default=0.0)
    s.add_argument("--no-memory-watchdog", action="store_true",
                   help="do not poll free device / host memory (soft floor pauses admission, hard floor trips the fault latch)")
    s.add_argument("--high-speed-swap-gb", type=float, default=0.0, help="file-backed KV tier below the host tier")
    s.add_argument("--high-speed-swap-path", default="", help="directory of the swap file (an NVMe mount)")
    s.add_argument("--quantization", default="auto", choices=["auto", "none", "fp8_block", "nvfp4"],
                   help="auto: what the checkpoint ships; otherwise quantise high-precision weights at load")
    s.add_argument("--dtype", default=None)
    s.add_argument("--rank", type=int, default=None)
    s.add_argument("--world-size", type=int, default=None)
    s.add_argument("--tp-size", type=int, default=0)
    s.add_argument("--ep-size", type=int, default=0)
    s.add_argument("--master-addr", default=None)
    s.add_argument("--master-port", type=int, default=None)
    s.add_argument("--comm", default="p2p", choices=["p2p", "nccl"], help="GPU collectives: peer-memory kernels or the NCCL baseline")
    s.add_argument("--no-cuda-graphs", action="store_true")
    s.add_argument("--tool-call-parser", default=None)
    s.add_argument("--disable-thinking", action="store_true")
    s.add_argument("--max-thinking-budget", type=int, default=0)
    s.add_argument("--request-timeout", type=float, default=0.0)
    s.add_argument("--require-auth", action="store_true")
    s.add_argument("--api-key", action="append", default=[])
    s.add_argument("--rate-limit-rpm", type=float, default=0.0)
    s.add_argument("--lora-adapter", action="append", default=[], help="name=path (repeatable)")
    s.add_argument("--seed", type=int, default=0)
    s.add_argument("--profile", action="store_true", help="per-phase timers and launch trace on /serve-config")
    s.add_argument("--dump", default=None, help="directory receiving one JSON file per request")
    s.add_argument("--context-compaction", action="store_true",
                   help="elide / drop old chat turns so that an over-long conversation fits the context window")
    s.add_argument("--no-output-sanitizer", action="store_true",
                   help="do not treat leaked chat-template markers in the output text as end of turn")
    s.add_argument("--loop-guard", action="store_true", help="end a generation whose output repeats with a short period")
    s.add_argument("--loop-guard-span", type=int, default=128, help="tokens that must be periodic before the guard fires")
    s.add_argument("--check-kernels", action="store_true", help="run the kernel self-test before serving")
    s.add_argument("--dry-run", action="store_true", help="resolve everything, print the plan, do not load a model")

    b = sub.add_parser("benchmark", help="run a benchmark against a running server or in-process")
    b.add_argument("suite", choices=["concurrency-sweep", "ttft", "decode-floor", "kat-equality", "ssm-poison", "microbench"])
    b.add_argument("--url", default=None, help="base URL of a running server; omit to run in-process")
    b.add_argument("--model", default="preset:tiny-dense")
    b.add_argument("--isl", type=int, default=128)
    b.add_argument("--osl", type=int, default=1024)
    b.add_argument("--concurrency", default="1,2,4,8,16,32,64,128")
    b.add_argument("--reps", type=int, default=3)
    b.add_argument("--warmup", type=int, default=1)
    b.add_argument("--out", default=None)
    b.add_argument("--device", default=None)

    d = sub.add_parser("doctor", help="report hardware, kernel library and environment health")
    d.add_argument("--json", action="store_true")

    r = sub.add_parser("recipes", help="list built-in recipes or print the argv of one")
    r.add_argument("recipe", nargs="?")
    r.add_argument("--sync", metavar="INDEX_URL", help="fetch the recipes an index lists (https:// or file://) into the local recipe directory")
    r.add_argument("--dest", default=None, help="directory for --sync (default: $ATLAS_RECIPES_DIR or ~/.cache/atlas_b200/recipes)")
    return ap


# ----------------------------------------------------------------------------------------------------- serve
def resolve_serve_args(argv: List[str]):
    """Parse ``serve`` arguments with recipe defaults layered under explicit flags."""
    ap = build_parser()
    args = ap.parse_args(["serve"] + argv)
    recipe = None
    if args.recipe:
        from . import recipes
        recipe = recipes.resolve(args.recipe)
        layered = ["serve"] + recipe.argv()[1:] + argv
        args = ap.parse_args(layered)
        if not args.model:
            args.model = recipe.model
    if not args.model:
        ap.error("serve needs a model (or a --recipe that names one)")
    return args, recipe


def _engine_config(args, mcfg):
    from .config import EngineConfig
    prefix = args.enable_prefix_caching if args.enable_prefix_caching is not None else True
    return EngineConfig(max_seq_len=min(args.max_seq_len, max(mcfg.max_position_embeddings, 1)), block_size=args.block_size,
                        kv_cache_dtype=args.kv_cache_dtype, dcut_ratio=args.dcut_ratio,
                        mtp_draft_vocab=getattr(args, "mtp_vocab", 0), mtp_vocab_rank=getattr(args, "mtp_vocab_rank", "id"),
                        sparse_attention_blocks=args.sparse_attention_blocks,
                        kv_high_precision_layers=tuple(int(v) for v in args.kv_high_precision_layers.split(",") if v.strip()),
                        gpu_memory_utilization=args.gpu_memory_utilization,
                        num_kv_blocks=args.num_kv_blocks, max_num_seqs=args.max_num_seqs, max_batch_size=args.max_batch_size,
                        max_prefill_tokens=args.max_prefill_tokens, scheduling_policy=args.scheduling_policy,
                        tbt_deadline_ms=args.tbt_deadline_ms, enable_prefix_caching=prefix,
                        speculative=args.speculative,
                        num_drafts=args.num_drafts or (1 if args.speculative else (3 if (args.ngram_speculative or args.self_speculative) else 0)),
                        ngram_speculative=args.ngram_speculative, ngram_max=args.ngram_max, ngram_min=args.ngram_min,
                        self_speculative=args.self_speculative, self_spec_keep=args.self_spec_keep,
                        mtp_gate=True if args.mtp_gate is None else args.mtp_gate, ssm_cache_slots=args.ssm_cache_slots,
                        ssm_checkpoint_interval=args.ssm_checkpoint_interval, swap_space_gb=args.swap_space_gb, disk_swap_gb=args.high_speed_swap_gb,
                        disk_swap_path=args.high_speed_swap_path,
                        use_cuda_graphs=not args.no_cuda_graphs, tp_size=max(1, args.tp_size), ep_size=max(1, args.ep_size),
                        seed=args.seed, request_timeout_s=args.request_timeout)


def load_for_serving(args, pctx, device):
    """Model + tokenizer path from ``args.model``."""
    from .config import PRESETS, QuantConfig
    from .models import build_model
    if args.model.startswith("preset:"):
        name = args.model.split(":", 1)[1]
        if name not in PRESETS:
            raise SystemExit(f"unknown preset '{name}'; known: {', '.join(sorted(PRESETS))}")
        mcfg = PRESETS[name]()
        if args.quantization not in ("auto",):
            mcfg.quant = QuantConfig(method=args.quantization) if args.quantization != "none" else QuantConfig()
        if args.dtype:
            mcfg.dtype = args.dtype
        elif device.type == "cpu":
            mcfg.dtype = "float32"
        elif mcfg.dtype == "float32":
            mcfg.dtype = "bfloat16"          # the GPU kernels take bf16 activations; the tiny presets default to fp32
        mcfg.max_position_embeddings = max(mcfg.max_position_embeddings, min(args.max_seq_len, 1 << 17))
        model = build_model(mcfg, pctx, device=device).init_random(args.seed, max_pos=min(args.max_seq_len, mcfg.max_position_embeddings) + 64)
        return model, None
    from .config import ModelConfig
    from .loader import Checkpoint, load_weights
    from .utils.model_resolver import ModelNotFound, resolve_model
    try:
        args.model = resolve_model(args.model)          # hub-style ids resolve to a local snapshot (offline)
    except ModelNotFound as e:
        raise SystemExit(str(e))
    mcfg = ModelConfig.from_pretrained(args.model)
    if args.quantization not in ("auto", "none"):
        mcfg.quant = QuantConfig(method=args.quantization)
    if args.dtype:
        mcfg.dtype = args.dtype
    elif device.type == "cpu":
        mcfg.dtype = "float32"
    model = build_model(mcfg, pctx, device=device)
    load_weights(model, Checkpoint(args.model))
    model.finalize(min(args.max_seq_len, mcfg.max_position_embeddings) + 64)
    return model, args.model


def cmd_serve(argv: List[str]) -> int:
    args, recipe = resolve_serve_args(argv)
    if recipe is not None:
        recipe.export_env()
    for k, v in (("RANK", args.rank), ("WORLD_SIZE", args.world_size), ("MASTER_ADDR", args.master_addr), ("MASTER_PORT", args.master_port)):
        if v is not None:
            os.environ[k] = str(v)
    if args.rank is not None and "LOCAL_RANK" not in os.environ:
        os.environ["LOCAL_RANK"] = str(args.rank)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if recipe is not None and world < recipe.min_ranks:
        raise SystemExit(f"recipe {recipe.id} needs {recipe.min_ranks} ranks, this launch has {world}")
    plan = {"model": args.model, "recipe": recipe.id if recipe else None, "world_size": world,
            "tp_size": args.tp_size or None, "ep_size": args.ep_size or None, "port": args.port,
            "flags": {k: v for k, v in vars(args).items() if k not in ("cmd", "api_key")}}
    if args.dry_run:
        print(json.dumps(plan, indent=1, default=str))
        return 0

    import torch

    from .engine import LLMEngine
    from .parallel import init_distributed
    t0 = time.time()
    topo, pctx, device = init_distributed(tp_size=args.tp_size, ep_size=args.ep_size)
    log = (lambda *a: print(f"[atlas rank {topo.rank}]", *a, file=sys.stderr, flush=True))
    control = None
    symm = None
    if topo.world_size > 1:
        from .parallel.worker import make_control
        control = make_control(timeout_s=float(os.environ.get("ATLAS_CONTROL_TIMEOUT_S", "30")))
        if device.type == "cuda" and args.comm == "p2p":
            from .parallel.symm import SymmBackend
            symm = SymmBackend(pctx.comm, device)
            pctx.comm = symm
            if pctx.ep_comm is not None and topo.overlapping:
                pctx.ep_comm = symm
    if args.profile:
        from .utils.trace import TRACER
        TRACER.enable(True)
    if args.check_kernels and device.type == "cuda":
        from .utils.selfcheck import kernel_selftest
        kernel_selftest(device)
    model, tok_path = load_for_serving(args, pctx, device)
    log(f"model ready in {time.time() - t0:.1f}s on {device}")
    ecfg = _engine_config(args, model.cfg)
    engine = LLMEngine(model, ecfg)
    log(f"engine ready: {engine.pool.num_blocks} KV blocks of {ecfg.block_size} tokens")
    if device.type == "cuda" and not args.no_memory_watchdog:
        from .utils.watchdog import attach
        attach(engine).start()

    if control is not None and not control.is_leader:
        from .parallel.worker import worker_loop
        n = worker_loop(engine, control)
        log(f"follower stopped after {n} steps")
        return 0

    import uvicorn

    from .server.app import ServerState, create_app
    from .server.engine_async import AsyncEngine
    from .server.tokenizer import load_tokenizer
    target = engine
    if control is not None:
        from .parallel.worker import DistributedEngine
        target = DistributedEngine(engine, control)
    aeng = AsyncEngine(target)
    tokenizer = load_tokenizer(tok_path, model.cfg.vocab_size)
    keys = list(args.api_key) + [k for k in os.environ.get("ATLAS_API_KEYS", "").split(",") if k]
    state = ServerState(aeng, tokenizer, args.served_model_name or os.path.basename(args.model.rstrip("/")) or args.model,
                        {"api_keys": keys if (keys or args.require_auth) else None, "rate_limit_rpm": args.rate_limit_rpm,
                         "tool_call_parser": args.tool_call_parser, "no_logit_pipeline": args.no_logit_pipeline,
                         "think_confidence_streak": args.think_confidence_streak, "margin_counter": args.margin_counter, "disable_thinking": args.disable_thinking,
                         "max_thinking_budget": args.max_thinking_budget, "dump": args.dump, "profile": args.profile, "loop_guard": args.loop_guard, "no_output_sanitizer": args.no_output_sanitizer, "context_compaction": args.context_compaction,
                         "loop_guard_span": args.loop_guard_span,
                         "serve_plan": plan})
    for spec in args.lora_adapter:
        name, _, path = spec.partition("=")
        state.adapters[name] = {"path": path, "slot": target.load_adapter(name, path)}      # followers get it with the first plan
    app = create_app(state)
    aeng.start()
    try:
        uvicorn.run(app, host=args.bind, port=args.port, log_level="warning")
    finally:
        aeng.shutdown(drain=True, timeout_s=10.0)
        if control is not None:
            target.shutdown()
        if symm is not None:
            symm.close()
        if topo.world_size > 1:
            torch.distributed.destroy_process_group()
    return 0


# ----------------------------------------------------------------------------------------------------- doctor
def doctor_report() -> dict:
    """Everything an operator needs before serving: GPU, driver, kernel library, peer access, Python deps."""
    import importlib

    from .utils.hardware import fingerprint
    rep = {"hardware": fingerprint(), "checks": []}

    def check(name, fn):
        try:
            ok, detail = fn()
        except Exception as e:     # noqa: BLE001 - a doctor reports, it does not crash
            ok, detail = False, f"{e.__class__.__name__}: {e}"
        rep["checks"].append({"name": name, "ok": bool(ok), "detail": detail})

    def kernels():
        from .ops import cuda as K
        return os.path.exists(K.LIB_PATH), K.LIB_PATH

    def gpu():
        import torch
        if not torch.cuda.is_available():
            return False, "no CUDA device visible (CPU reference path only)"
        cc = torch.cuda.get_device_capability(0)
        return cc[0] == 10, f"{torch.cuda.get_device_name(0)} sm_{cc[0]}{cc[1]} x{torch.cuda.device_count()}"

    def peers():
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        if n < 2:
            return True, "single GPU"
        bad = [(i, j) for i in range(n) for j in range(n) if i != j and not torch.cuda.can_device_access_peer(i, j)]
        return not bad, "all pairs peer-accessible" if not bad else f"no peer access: {bad[:4]}"

    def deps():
        missing = [m for m in ("fastapi", "uvicorn", "safetensors", "tokenizers", "jinja2", "yaml") if importlib.util.find_spec(m) is None]
        return not missing, "ok" if not missing else "missing: " + ", ".join(missing)

    def grammar():
        return True, "xgrammar" if importlib.util.find_spec("xgrammar") else "built-in JSON matcher (xgrammar not installed)"

    check("kernel library", kernels)
    check("gpu", gpu)
    check("peer access", peers)
    check("python deps", deps)
    check("grammar backend", grammar)
    rep["ok"] = all(c["ok"] for c in rep["checks"] if c["name"] in ("kernel library", "python deps"))
    return rep


def cmd_doctor(argv: List[str]) -> int:
    args = build_parser().parse_args(["doctor"] + argv)
    rep = doctor_report()
    if args.json:
        print(json.dumps(rep, indent=1, default=str))
    else:
        for c in rep["checks"]:
            print(f"[{'ok' if c['ok'] else '!!'}] {c['name']}: {c['detail']}")
    return 0 if rep["ok"] else 1


# ----------------------------------------------------------------------------------------------------- benchmark / recipes
def cmd_benchmark(argv: List[str]) -> int:
    args = build_parser().parse_args(["benchmark"] + argv)
    if args.suite == "microbench":
        from .bench import microbench
        sys.argv = ["microbench"]
        return microbench.main() or 0
    from .bench import ladder
    return ladder.main_from_args(args)


def cmd_recipes(argv: List[str]) -> int:
    from . import recipes
    args = build_parser().parse_args(["recipes"] + argv)
    if args.sync:
        for rid in recipes.sync(args.sync, args.dest):
            print(rid)
        return 0
    if not args.recipe:
        for rid, d in sorted(recipes.BUILTIN.items()):
            print(f"{rid:36s} ranks>={d.get('min_ranks', 1)}  {d.get('description', '')}")
        return 0
    print(" ".join(["serve"] + recipes.resolve(args.recipe).argv()))
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        build_parser().parse_args(argv or ["--help"])
        return 0
    cmd, rest = argv[0], argv[1:]
    table = {"serve": cmd_serve, "benchmark": cmd_benchmark, "doctor": cmd_doctor, "recipes": cmd_recipes}
    if cmd not in table:
        build_parser().parse_args(argv)
        return 2
    return table[cmd](rest)
