"""Serving benchmarks and gates: concurrency sweep, TTFT cold/warm, decode floor, order-independence (KAT equality) and
recurrent-state poisoning.

Two drivers share the measurement code:

* in-process (`EngineDriver`): requests go through :class:`~atlas_b200.engine.LLMEngine` directly; per-token arrival
  times are taken from the step loop, so TTFT / TPOT are engine-side numbers;
* HTTP (`HttpDriver`): a streaming OpenAI client (aiohttp, SSE) against a running server; the numbers are the
  client's, which is what the published ladder reports.

Reference parity: ``crates/avarok-plugin/src/benchmarks/{concurrency,ttft,decode_floor,kat_equality,ssm_poison}.rs``
(metric definitions: fire C streaming requests at once per (ISL x C) cell, aggregate output tok/s of the batch, client
TTFT / TPOT / E2E percentiles, mean of timed repetitions after warm-up; cold TTFT = unique prefix per sample, warm =
primed identical prompt; KAT equality = byte-exact outputs whatever shares the batch; SSM poison = byte-identical
replay after other traffic has run through the state slots and the prefix cache).
"""
from __future__ import annotations

import asyncio
import json
import statistics
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


def pct(xs: Sequence[float], q: float) -> Optional[float]:
    if not xs:
        return None
    s = sorted(xs)
    i = min(len(s) - 1, max(0, int(round(q / 100.0 * (len(s) - 1)))))
    return s[i]


@dataclass
class RequestTrace:
    n_prompt: int
    t_submit: float
    t_first: Optional[float] = None
    t_done: Optional[float] = None
    tokens: List[int] = field(default_factory=list)
    text: str = ""

    @property
    def ttft(self) -> Optional[float]:
        return None if self.t_first is None else self.t_first - self.t_submit

    @property
    def tpot(self) -> Optional[float]:
        n = len(self.tokens)
        if self.t_first is None or self.t_done is None or n < 2:
            return None
        return (self.t_done - self.t_first) / (n - 1)


def summarise(traces: List[RequestTrace], wall: float) -> Dict[str, float]:
    out_tokens = sum(len(t.tokens) for t in traces)
    ttfts = [t.ttft * 1e3 for t in traces if t.ttft is not None]
    tpots = [t.tpot * 1e3 for t in traces if t.tpot is not None]
    e2es = [(t.t_done - t.t_submit) * 1e3 for t in traces if t.t_done is not None]
    return {"requests": len(traces), "output_tokens": out_tokens, "wall_s": wall,
            "agg_output_tok_s": out_tokens / wall if wall > 0 else 0.0,
            "ttft_ms_p50": pct(ttfts, 50), "ttft_ms_p90": pct(ttfts, 90), "ttft_ms_p99": pct(ttfts, 99),
            "tpot_ms_p50": pct(tpots, 50), "tpot_ms_p90": pct(tpots, 90), "tpot_ms_p99": pct(tpots, 99),
            "e2e_ms_p50": pct(e2es, 50), "e2e_ms_p90": pct(e2es, 90), "e2e_ms_p99": pct(e2es, 99)}


# ----------------------------------------------------------------------------------------------------- drivers
class EngineDriver:
    """Runs a batch of token-id prompts through an in-process engine."""

    def __init__(self, engine):
        self.engine = engine
        self.vocab = engine.mcfg.vocab_size

    def run_batch(self, prompts: List[List[int]], max_tokens: int, samplings=None, seed: Optional[int] = 42) -> List[RequestTrace]:
        from ..sampling import SamplingParams
        eng = self.engine
        traces: Dict[str, RequestTrace] = {}
        t0 = time.perf_counter()
        for i, p in enumerate(prompts):
            sp = samplings[i] if samplings else SamplingParams(max_tokens=max_tokens, temperature=0.0, ignore_eos=True, seed=seed)
            rid = eng.add_request(p, sp)
            traces[rid] = RequestTrace(len(p), t0)
        order = list(traces)
        while eng.has_unfinished():
            outs = eng.step()
            now = time.perf_counter()
            for o in outs:
                tr = traces.get(o.request_id)
                if tr is None:
                    continue
                if o.new_tokens:
                    if tr.t_first is None:
                        tr.t_first = now
                    tr.tokens.extend(o.new_tokens)
                if o.finished:
                    tr.t_done = now
        return [traces[r] for r in order]


class HttpDriver:
    """Streaming OpenAI-completions client; prompts are sent as token id arrays."""

    def __init__(self, url: str, model: str = "default", api_key: Optional[str] = None):
        self.url, self.model, self.api_key = url.rstrip("/"), model, api_key

    async def _one(self, session, prompt: List[int], max_tokens: int, trace: RequestTrace, seed) -> None:
        body = {"model": self.model, "prompt": prompt, "max_tokens": max_tokens, "temperature": 0.0, "stream": True,
                "ignore_eos": True, "seed": seed, "return_token_ids": True}
        headers = {"Authorization": f"Bearer {self.api_key}"} if self.api_key else {}
        async with session.post(self.url + "/v1/completions", json=body, headers=headers) as resp:
            resp.raise_for_status()
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data:"):
                    continue
                data = line[5:].strip()
                if data == "[DONE]":
                    break
                ev = json.loads(data)
                ch = (ev.get("choices") or [{}])[0]
                ids = ch.get("token_ids") or []
                txt = ch.get("text") or ""
                if ids or txt:
                    if trace.t_first is None:
                        trace.t_first = time.perf_counter()
                    trace.tokens.extend(ids if ids else [0] * max(1, len(txt.split())))
                    trace.text += txt
        trace.t_done = time.perf_counter()

    def run_batch(self, prompts: List[List[int]], max_tokens: int, samplings=None, seed: Optional[int] = 42) -> List[RequestTrace]:
        import aiohttp

        async def go():
            t0 = time.perf_counter()
            traces = [RequestTrace(len(p), t0) for p in prompts]
            timeout = aiohttp.ClientTimeout(total=3600)
            async with aiohttp.ClientSession(timeout=timeout) as s:
                await asyncio.gather(*[self._one(s, p, max_tokens, tr, seed) for p, tr in zip(prompts, traces)])
            return traces
        return asyncio.run(go())


# ----------------------------------------------------------------------------------------------------- suites
def _rand_prompts(n: int, length: int, vocab: int, seed: int, shared_prefix: int = 0) -> List[List[int]]:
    import torch
    g = torch.Generator().manual_seed(seed)
    prefix = torch.randint(3, vocab, (shared_prefix,), generator=g).tolist() if shared_prefix else []
    return [prefix + torch.randint(3, vocab, (length - shared_prefix,), generator=g).tolist() for _ in range(n)]


def concurrency_sweep(driver, vocab: int, isl: int = 128, osl: int = 1024, ladder: Sequence[int] = (1, 2, 4, 8, 16, 32, 64, 128),
                      reps: int = 3, warmup: int = 1, seed: int = 42) -> List[dict]:
    """One row per rung: mean over ``reps`` of the aggregate output tok/s, medians of the latency percentiles."""
    rows = []
    for c in ladder:
        cells = []
        for r in range(warmup + reps):
            prompts = _rand_prompts(c, isl, vocab, seed * 1000 + c * 10 + r)      # fresh prompts: no prefix-cache help
            t0 = time.perf_counter()
            traces = driver.run_batch(prompts, osl, seed=seed)
            cell = summarise(traces, time.perf_counter() - t0)
            if r >= warmup:
                cells.append(cell)
        row = {"isl": isl, "osl": osl, "concurrency": c, "reps": reps,
               "agg_output_tok_s": statistics.mean(x["agg_output_tok_s"] for x in cells)}
        for k in ("ttft_ms_p50", "ttft_ms_p90", "ttft_ms_p99", "tpot_ms_p50", "tpot_ms_p90", "e2e_ms_p50"):
            vals = [x[k] for x in cells if x[k] is not None]
            row[k] = statistics.median(vals) if vals else None
        rows.append(row)
    return rows


def ttft_gate(driver, vocab: int, lengths: Sequence[int] = (256, 1024, 4096), repeats: int = 12, seed: int = 7,
              ceilings: Optional[Dict[str, float]] = None) -> dict:
    """Cold: a unique prompt per sample.  Warm: the same prompt again after a priming request (prefix-cache hit)."""
    cold, warm = [], []
    for n in lengths:
        for r in range(repeats):
            p = _rand_prompts(1, n, vocab, seed * 100000 + n * 100 + r)
            cold.append(driver.run_batch(p, 2)[0].ttft * 1e3)
            warm.append(driver.run_batch(p, 2)[0].ttft * 1e3)       # primed by the cold sample just above
    res = {"cold_ms_median": statistics.median(cold), "cold_ms_p90": pct(cold, 90),
           "warm_ms_median": statistics.median(warm), "warm_ms_p90": pct(warm, 90), "samples": len(cold)}
    if ceilings:
        res["pass"] = all(res[k] <= v for k, v in ceilings.items() if k in res)
    return res


def decode_floor(driver, vocab: int, min_tokens: int = 750, runs: int = 3, floor_tok_s: Optional[float] = None) -> dict:
    """Single-stream decode rate over long generations (first token excluded)."""
    rates = []
    for r in range(runs):
        tr = driver.run_batch(_rand_prompts(1, 32, vocab, 900 + r), min_tokens)[0]
        rates.append((len(tr.tokens) - 1) / (tr.t_done - tr.t_first))
    res = {"decode_tok_s_min": min(rates), "decode_tok_s_median": statistics.median(rates), "runs": runs}
    if floor_tok_s is not None:
        res["pass"] = res["decode_tok_s_min"] >= floor_tok_s
    return res


def kat_equality(driver, vocab: int, n: int = 8, isl: int = 48, osl: int = 24, sampled: bool = True) -> dict:
    """Order independence: each request alone must produce byte-identical tokens to the same request inside a full
    batch and inside a batch submitted in reverse order (seeded sampling included)."""
    from ..sampling import SamplingParams
    prompts = _rand_prompts(n, isl, vocab, 4242)

    def sp(i):
        if sampled and i % 2:
            return SamplingParams(max_tokens=osl, temperature=0.8, top_p=0.9, top_k=40, seed=1000 + i, ignore_eos=True)
        return SamplingParams(max_tokens=osl, temperature=0.0, ignore_eos=True)

    together = [t.tokens for t in driver.run_batch(prompts, osl, [sp(i) for i in range(n)])]
    rev = [t.tokens for t in driver.run_batch(prompts[::-1], osl, [sp(i) for i in range(n)][::-1])][::-1]
    solo = [driver.run_batch([prompts[i]], osl, [sp(i)])[0].tokens for i in range(n)]
    bad = [i for i in range(n) if not (together[i] == rev[i] == solo[i])]
    return {"requests": n, "mismatching": bad, "pass": not bad}


def ssm_poison(driver, vocab: int, isl: int = 96, osl: int = 24, noise_rounds: int = 3, noise_batch: int = 6) -> dict:
    """State poisoning: a probe's output must not change after unrelated traffic has cycled through the recurrent-state
    slots, the snapshot slots and the prefix cache — neither on a prefix-cache hit nor on a cold replay."""
    probe = _rand_prompts(1, isl, vocab, 31337)
    first = driver.run_batch(probe, osl)[0].tokens
    for r in range(noise_rounds):
        noise = _rand_prompts(noise_batch, isl + 16 * r, vocab, 5000 + r, shared_prefix=32 if r % 2 else 0)
        driver.run_batch(noise + probe[:1] * (r % 2), osl)
    again = driver.run_batch(probe, osl)[0].tokens
    extended = driver.run_batch([probe[0] + first[:4]], osl - 4)[0].tokens       # continue from a longer cached prefix
    ok_ext = extended == first[4:]
    return {"pass": first == again and ok_ext, "replay_equal": first == again, "extended_equal": ok_ext}


# ----------------------------------------------------------------------------------------------------- CLI glue
def _inprocess_engine(model_spec: str, device: Optional[str], max_len: int, concurrency: int):
    import torch

    from ..config import PRESETS, EngineConfig
    from ..engine import LLMEngine
    from ..models import build_model
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    if model_spec.startswith("preset:"):
        mcfg = PRESETS[model_spec.split(":", 1)[1]]()
        if dev.type == "cpu":
            mcfg.dtype = "float32"
        elif mcfg.dtype == "float32":
            mcfg.dtype = "bfloat16"          # the GPU kernels take bf16 activations; the tiny presets default to fp32
        mcfg.max_position_embeddings = max(mcfg.max_position_embeddings, max_len + 64)
        model = build_model(mcfg, device=dev).init_random(0, max_pos=max_len + 64)
    else:
        from ..loader import load_model
        model = load_model(model_spec, device=dev, dtype="float32" if dev.type == "cpu" else None, max_pos=max_len + 64)
    blocks = (max_len // 16 + 2) * max(concurrency, 1) + 64
    ecfg = EngineConfig(max_seq_len=max_len + 32, max_num_seqs=max(concurrency, 1), max_batch_size=max(concurrency, 1),
                        num_kv_blocks=blocks if dev.type == "cpu" else None)
    return LLMEngine(model, ecfg)


def main_from_args(args) -> int:
    ladder = [int(x) for x in str(args.concurrency).split(",") if x]
    if args.url:
        import urllib.request
        with urllib.request.urlopen(args.url.rstrip("/") + "/v1/models", timeout=10) as r:
            card = json.loads(r.read())["data"][0]
        driver, vocab = HttpDriver(args.url, card["id"]), int(card.get("vocab_size", 32000))
    else:
        eng = _inprocess_engine(args.model, args.device, args.isl + args.osl, max(ladder))
        driver, vocab = EngineDriver(eng), eng.mcfg.vocab_size
    if args.suite == "concurrency-sweep":
        res = {"suite": args.suite, "rows": concurrency_sweep(driver, vocab, args.isl, args.osl, ladder, args.reps, args.warmup)}
    elif args.suite == "ttft":
        res = {"suite": args.suite, **ttft_gate(driver, vocab, lengths=(min(256, args.isl), args.isl), repeats=args.reps)}
    elif args.suite == "decode-floor":
        res = {"suite": args.suite, **decode_floor(driver, vocab, min_tokens=args.osl, runs=args.reps)}
    elif args.suite == "kat-equality":
        if args.url:
            raise SystemExit("kat-equality needs per-request sampling control: run it in-process")
        res = {"suite": args.suite, **kat_equality(driver, vocab)}
    elif args.suite == "ssm-poison":
        res = {"suite": args.suite, **ssm_poison(driver, vocab)}
    else:
        raise SystemExit(f"unknown suite {args.suite}")
    text = json.dumps(res, indent=1)
    print(text)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text)
    return 0 if res.get("pass", True) else 1
