"""Where one engine step spends its device time: every kernel-launching call of the op layer is followed by a CUDA
event, and the gaps between consecutive events are summed per kernel name (anything else that ran on the stream in
between, e.g. a framework copy, is charged to the call that follows it).

    python -m atlas_b200.bench.step_profile --model llama3-8b --batch 128 --ctx 1152            # decode step
    python -m atlas_b200.bench.step_profile --model qwen3-30b-a3b --batch 128 --ctx 2304
    python -m atlas_b200.bench.step_profile --model llama3-8b --prefill 8192                    # one prefill chunk

Eager launches (no CUDA graph), so launch gaps of a host-bound step show up inside the numbers: read the shares and the
sum against the graph-replayed step time that ``bench.py`` reports.

Reference parity: ``crates/spark-runtime/src/launch_trace.rs`` (per-launch records aggregated by kernel).
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict

import torch


def run(model_name: str, batch: int, ctx: int, prefill: int, steps: int, block_size: int = 16, prefill_seqs: int = 1):
    from atlas_b200.config import PRESETS
    from atlas_b200.models import build_model
    from atlas_b200.models.batch import ForwardBatch
    from atlas_b200.ops import cuda as K
    K.load()
    dev = "cuda"
    cfg = PRESETS[model_name]()
    total = (ctx + 1) if not prefill else prefill
    cfg.max_position_embeddings = max(4096, total + 16)
    model = build_model(cfg, device=dev).init_random(0, max_pos=total + 16)
    nseq = batch if not prefill else max(1, prefill_seqs)
    if prefill:
        total = prefill // nseq                      # the chunk is `prefill_seqs` prompts of equal length
    per = (total + block_size - 1) // block_size + 1
    cache = model.alloc_cache(nseq * per + 8, block_size, torch.float8_e4m3fn, state_slots=nseq + 1)
    tables = [list(range(i * per, (i + 1) * per)) for i in range(nseq)]
    g = torch.Generator().manual_seed(0)
    if prefill:
        toks = [torch.randint(0, cfg.vocab_size, (total,), generator=g).tolist() for _ in range(nseq)]
        mk = lambda: ForwardBatch.build(toks, [0] * nseq, tables, block_size, device=dev, state_slots=list(range(nseq)),
                                        has_state=[False] * nseq)
    else:
        toks = [[int(torch.randint(0, cfg.vocab_size, (1,), generator=g))] for _ in range(batch)]
        mk = lambda: ForwardBatch.build(toks, [ctx] * batch, tables, block_size, device=dev,
                                        state_slots=list(range(batch)), has_state=[True] * batch)
    def logits(h, fb):
        # like the engine: only the last row of every sequence goes through the output projection
        if prefill:
            return model.compute_logits(h, (fb.query_start_loc[1:] - 1).long())
        return model.compute_logits(h)
    for _ in range(2):
        logits(model.forward(mk_fb := mk(), cache), mk_fb)
    torch.cuda.synchronize()
    agg = defaultdict(lambda: [0.0, 0])
    step_ms = []
    for _ in range(steps):
        fb = mk()
        torch.cuda.synchronize()
        K.device_marks = []
        t0 = torch.cuda.Event(enable_timing=True)
        t0.record()
        logits(model.forward(fb, cache), fb)
        marks, K.device_marks = K.device_marks, None
        torch.cuda.synchronize()
        prev = t0
        for name, ev in marks:
            a = agg[name]
            a[0] += prev.elapsed_time(ev) * 1e3
            a[1] += 1
            prev = ev
        step_ms.append(t0.elapsed_time(marks[-1][1]))
    rows = sorted(((n, v[0] / steps, v[1] // steps) for n, v in agg.items()), key=lambda r: -r[1])
    tot = sum(r[1] for r in rows)
    out = {"model": model_name, "mode": "prefill" if prefill else "decode", "batch": nseq, "ctx": ctx, "tokens": prefill or batch,
           "step_ms_eager": round(sum(step_ms) / len(step_ms), 3), "launches_per_step": sum(r[2] for r in rows),
           "kernels": [{"name": n, "us": round(us, 1), "calls": c, "share": round(us / tot, 3)} for n, us, c in rows]}
    assert K.check_status() == 0
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--prefill", type=int, default=0, help="profile one prefill chunk of this many tokens instead of a decode step")
    ap.add_argument("--prefill-seqs", type=int, default=1, help="split the prefill chunk into this many equal prompts")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    res = run(a.model, a.batch, a.ctx, a.prefill, a.steps, prefill_seqs=a.prefill_seqs)
    print(json.dumps({k: v for k, v in res.items() if k != "kernels"}))
    for k in res["kernels"]:
        print(f'{k["name"]:<28} {k["calls"]:>5} x  {k["us"]:>10.1f} us  {100 * k["share"]:5.1f} %')
    if a.out:
        with open(a.out, "w") as f:
            json.dump(res, f, indent=1)


if __name__ == "__main__":
    main()
