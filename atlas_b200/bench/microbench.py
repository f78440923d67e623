"""Kernel micro-benchmarks with roofline fractions.

``python -m atlas_b200.bench.microbench [--model llama3-8b] [--out FILE]`` times every hot kernel on the
shapes the named model produces (decode batch and prefill chunk), with CUDA events on the launching
stream, three warm-up runs, an L2 flush (a 256 MiB write) between timed runs, and prints achieved GB/s /
TFLOP/s and the fraction of the measured peaks (``MEASURED_PEAKS.json`` next to the repository root when
present, else the documented fallback figures).

Reference counterpart: the kernel micro-benchmark table of ``book/src/operations/benchmarks.md:67-102``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from typing import Callable, Dict, List, Optional

import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks() -> Dict[str, float]:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    d = dict(FALLBACK_PEAKS)
    d["source"] = "fallback"
    return d


class Timer:
    def __init__(self, device="cuda", use_graph: bool = True):
        self.use_graph = use_graph
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def time(self, fn: Callable[[], None], iters: int = 7, warmup: int = 3) -> float:
        """Median milliseconds of ``fn`` with a cold L2.  ``fn`` is captured into a CUDA graph first so that
        host-side launch cost (Python, descriptor lookup, allocator) is not part of the number."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if self.use_graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            fn = g.replay
            fn()
            torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            self.flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            fn()
            e.record()
            e.synchronize()
            ts.append(s.elapsed_time(e))
        return statistics.median(ts)


def run(model: str = "llama3-8b", decode_batch: int = 128, ctx: int = 1152, chunk: int = 8192,
        only: Optional[str] = None) -> List[dict]:
    from atlas_b200 import quant as Q
    from atlas_b200.config import PRESETS
    from atlas_b200.models.batch import ForwardBatch
    from atlas_b200.ops import cuda as K
    from atlas_b200.ops import reference as ref
    K.load()
    cfg = PRESETS[model]()
    peaks = load_peaks()
    dev = "cuda"
    T = Timer(dev)
    rows: List[dict] = []

    def add(name, ms, bytes_=0, flops=0, note=""):
        r = {"kernel": name, "ms": round(ms, 4), "note": note}
        if bytes_:
            gbs = bytes_ / ms / 1e6
            r["GB/s"] = round(gbs, 1)
            r["frac_hbm"] = round(gbs / peaks["hbm_gbs"], 3)
        if flops:
            tf = flops / ms / 1e9
            r["TFLOP/s"] = round(tf, 1)
            r["frac_bf16_peak"] = round(tf / peaks["bf16_tflops"], 3)
        rows.append(r)
        print(json.dumps(r), flush=True)

    H, I = cfg.hidden_size, cfg.intermediate_size
    qkv_n = cfg.q_size + 2 * cfg.kv_size
    gemms = [("qkv", qkv_n, H), ("o", H, cfg.q_size), ("gate_up", 2 * I, H), ("down", H, I)]
    if not only or only == "gemm":
        for M in (decode_batch, chunk):
            x = torch.randn(M, max(H, I), device=dev).bfloat16()
            for name, N, Kd in gemms:
                w = torch.randn(N, Kd, device=dev) * 0.02
                wq, ws = Q.quantize_fp8_block(w)
                del w
                xq, xs = K.quant_fp8(x[:, :Kd].contiguous())
                out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
                ms = T.time(lambda: K.gemm_fp8_block(xq, xs, wq, ws, out=out))
                bn, sp = K.gemm_plan(M, N, Kd, 1, 148)
                add(f"gemm_fp8 {name} M={M} N={N} K={Kd}", ms, bytes_=N * Kd + M * Kd + 2 * M * N, flops=2 * M * N * Kd,
                    note=f"block_n={bn} splits={sp}")
                # fused epilogues of the same shape: SwiGLU + FP8 quant (gate_up), residual + norm weight + FP8 quant (o, down)
                if name == "gate_up" and (N // 2) % 128 == 0:
                    ms = T.time(lambda: K.gemm_fp8_fused(xq, xs, wq, ws, mode=1))
                    add(f"gemm_fp8+swiglu+quant {name} M={M}", ms, bytes_=N * Kd + M * Kd + M * N // 2, flops=2 * M * N * Kd)
                if name in ("o", "down") and N % 128 == 0:
                    res = torch.randn(M, N, device=dev).bfloat16()
                    nw = torch.ones(N, device=dev).bfloat16()
                    ms = T.time(lambda: K.gemm_fp8_fused(xq, xs, wq, ws, mode=2, residual=res, norm_w=nw))
                    add(f"gemm_fp8+residual+norm+quant {name} M={M}", ms, bytes_=N * Kd + M * Kd + 5 * M * N, flops=2 * M * N * Kd)
                # the library's FP8 GEMM (cuBLASLt through torch._scaled_mm, ONE scale per tensor: no 128x128 block fold)
                # and its bf16 GEMM on the same shape
                try:
                    one = torch.ones((), device=dev)
                    ms = T.time(lambda: torch._scaled_mm(xq, wq.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
                    add(f"library fp8 tensorwise (_scaled_mm) {name} M={M}", ms, bytes_=N * Kd + M * Kd + 2 * M * N,
                        flops=2 * M * N * Kd, note="no block scales: a lower bound the block-scaled kernel cannot reach")
                except Exception as exc:                                       # pragma: no cover
                    print(json.dumps({"kernel": f"_scaled_mm {name}", "error": repr(exc)[:200]}), flush=True)
                xb, wb = x[:, :Kd].contiguous(), torch.randn(N, Kd, device=dev).bfloat16()
                ms = T.time(lambda: torch.matmul(xb, wb.t()))
                add(f"library bf16 (cuBLAS) {name} M={M}", ms, bytes_=2 * (N * Kd + M * Kd + M * N), flops=2 * M * N * Kd)
                del wq, ws, wb
        # lm_head bf16
        M = decode_batch
        w = (torch.randn(cfg.vocab_size, H, device=dev) * 0.02).bfloat16()
        x = torch.randn(M, H, device=dev).bfloat16()
        out = torch.empty(M, cfg.vocab_size, dtype=torch.bfloat16, device=dev)
        ms = T.time(lambda: K.gemm_bf16(x, w, out=out))
        add(f"gemm_bf16 lm_head M={M} N={cfg.vocab_size} K={H}", ms, bytes_=2 * cfg.vocab_size * H + 2 * M * cfg.vocab_size,
            flops=2 * M * cfg.vocab_size * H)
        M = 4096
        x = torch.randn(M, H, device=dev).bfloat16()
        w2 = w[:8192]
        out = torch.empty(M, 8192, dtype=torch.bfloat16, device=dev)
        ms = T.time(lambda: K.gemm_bf16(x, w2, out=out))
        add(f"gemm_bf16 M={M} N=8192 K={H}", ms, flops=2 * M * 8192 * H, bytes_=2 * (M * H + 8192 * H + M * 8192))
        del w, w2

    if not only or "nvfp4" in only:
        # NVFP4 weight-only GEMM: packed weights (0.5 B) + block scales (1/16 B) per weight are the HBM traffic
        for M in (decode_batch, chunk):
            x = torch.randn(M, max(H, I), device=dev).bfloat16()
            for name, N, Kd in gemms:
                pk, bs, gs = Q.quantize_nvfp4(torch.randn(N, Kd, device=dev) * 0.02)
                xa = x[:, :Kd].contiguous()
                out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
                ms = T.time(lambda: K.gemm_nvfp4(xa, pk, bs, gs, out=out))
                add(f"gemm_nvfp4_w4a16 {name} M={M} N={N} K={Kd}", ms, bytes_=N * Kd * 9 // 16 + 2 * M * Kd + 2 * M * N,
                    flops=2 * M * N * Kd)
                del pk, bs, gs

    if not only or only == "w4a4":
        # NVFP4 x NVFP4 on the block-scaled tensor cores: the GEMM alone, and with the activation quantiser in front
        from atlas_b200.ops import cuda_fp4 as F4
        for M in (decode_batch, chunk):
            x = torch.randn(M, max(H, I), device=dev).bfloat16()
            for name, N, Kd in gemms:
                pk, bs, gs = Q.quantize_nvfp4(torch.randn(N, Kd, device=dev) * 0.02)
                wsf = F4.sf_atoms(bs)
                col = gs.expand(N).contiguous()
                xa = x[:, :Kd].contiguous()
                xq, xsf, xrs = F4.quant_nvfp4(xa)
                out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
                ms = T.time(lambda: F4.gemm_w4a4(xq, xsf, xrs, pk, wsf, col, out=out))
                add(f"gemm_nvfp4_w4a4 {name} M={M} N={N} K={Kd}", ms, bytes_=(N + M) * Kd * 9 // 16 + 2 * M * N, flops=2 * M * N * Kd)
                ms = T.time(lambda: F4.quant_nvfp4(xa))
                add(f"quant_nvfp4 {name} M={M} K={Kd}", ms, bytes_=M * Kd * 2 + M * Kd * 9 // 16)
                del pk, bs, gs, wsf

    if only and only.startswith("one4:"):
        # one NVFP4 x NVFP4 GEMM shape, few launches, no graph: the case to put under a profiler.  only = "one4:<name>:<M>"
        from atlas_b200.ops import cuda_fp4 as F4
        _, name, m_s = only.split(":")
        M = int(m_s)
        N, Kd = {n: (a, b) for n, a, b in gemms}[name]
        pk, bs, gs = Q.quantize_nvfp4(torch.randn(N, Kd, device=dev) * 0.02)
        wsf, col = F4.sf_atoms(bs), gs.expand(N).contiguous()
        xq, xsf, xrs = F4.quant_nvfp4(torch.randn(M, Kd, device=dev).bfloat16())
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        T.use_graph = False
        ms = T.time(lambda: F4.gemm_w4a4(xq, xsf, xrs, pk, wsf, col, out=out), iters=3, warmup=2)
        add(f"gemm_nvfp4_w4a4 {name} M={M} N={N} K={Kd}", ms, bytes_=(N + M) * Kd * 9 // 16 + 2 * M * N, flops=2 * M * N * Kd,
            note="eager launch")
        return rows

    if only and only.startswith("onefused:"):
        # one decode-size FP8 GEMM with its fused epilogue (o / down: residual + norm + FP8 quantisation, split-K through a
        # cluster; gate_up: SwiGLU), few eager launches: the case to put under a profiler.  only = "onefused:<name>:<M>"
        _, name, m_s = only.split(":")
        M = int(m_s)
        N, Kd = {n: (a, b) for n, a, b in gemms}[name]
        x = torch.randn(M, Kd, device=dev).bfloat16()
        wq, ws = Q.quantize_fp8_block(torch.randn(N, Kd, device=dev) * 0.02)
        xq, xs = K.quant_fp8(x)
        mode = 1 if name == "gate_up" else (2 if name in ("o", "down") else 0)
        res = torch.randn(M, N, device=dev).bfloat16()
        nw = torch.ones(N, device=dev).bfloat16()
        T.use_graph = False
        ms = T.time(lambda: K.gemm_fp8_fused(xq, xs, wq, ws, mode=mode, residual=res if mode == 2 else None,
                                             norm_w=nw if mode == 2 else None), iters=3, warmup=2)
        bn, sp = K.fused_block_n(mode, M, N, Kd, 148) if mode else K.gemm_plan(M, N, Kd, 1, 148)
        add(f"gemm_fp8 fused mode {mode} {name} M={M} N={N} K={Kd}", ms, bytes_=N * Kd + M * Kd + 2 * M * N, flops=2 * M * N * Kd,
            note=f"block_n={bn} splits={sp} (eager launch)")
        return rows

    if only and only.startswith("one:"):
        # one FP8 GEMM shape, few launches, no graph: the case to put under a profiler.  only = "one:<name>:<M>"
        _, name, m_s = only.split(":")
        M = int(m_s)
        N, Kd = {n: (a, b) for n, a, b in gemms}[name]
        x = torch.randn(M, Kd, device=dev).bfloat16()
        wq, ws = Q.quantize_fp8_block(torch.randn(N, Kd, device=dev) * 0.02)
        xq, xs = K.quant_fp8(x)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        T.use_graph = False
        ms = T.time(lambda: K.gemm_fp8_block(xq, xs, wq, ws, out=out), iters=3, warmup=2)
        bn, sp = K.gemm_plan(M, N, Kd, 1, 148)
        add(f"gemm_fp8 {name} M={M} N={N} K={Kd}", ms, bytes_=N * Kd + M * Kd + 2 * M * N, flops=2 * M * N * Kd,
            note=f"block_n={bn} splits={sp} (eager launch)")
        return rows

    if only == "stream":
        # What the memory system gives a weight stream on its own (bench/csrc/stream_probe.cu): tile copies through a ring, nothing
        # else, in the [N, K] weight layout (a tile's rows one leading dimension apart) and packed tile by tile.
        import ctypes as C
        from atlas_b200 import build as _build
        L = C.CDLL(_build.build_bench() if not os.path.exists(_build.BENCH_LIB) else _build.BENCH_LIB)
        L.atlas_probe_tma_stream.argtypes = [C.c_void_p, C.c_longlong] + [C.c_int] * 7 + [C.c_void_p, C.c_void_p, C.c_void_p]
        sink = torch.zeros(1, dtype=torch.int64, device=dev)
        buf = torch.empty(320 << 20, dtype=torch.uint8, device=dev)
        buf.random_(0, 255)
        K._dev(buf)
        for box, stages, tiles, kbs, ctas, pieces in ((64, 8, 96, 32, 96, 1), (64, 8, 148, 32, 148, 1), (64, 8, 148, 32, 148, 4),
                                                      (128, 6, 128, 32, 128, 1), (128, 6, 128, 32, 128, 4), (128, 6, 148, 32, 148, 1),
                                                      (128, 6, 148, 32, 148, 4), (128, 6, 148, 32, 148, 8), (128, 12, 148, 32, 148, 1),
                                                      (256, 4, 112, 32, 112, 1), (256, 4, 112, 32, 112, 8), (256, 6, 148, 32, 148, 1),
                                                      (256, 6, 148, 32, 148, 8), (128, 6, 148, 112, 148, 1), (128, 6, 148, 112, 148, 4),
                                                      # two and three CTAs per SM (the ring shrinks to fit)
                                                      (128, 6, 296, 32, 296, 1), (64, 8, 296, 32, 296, 1), (64, 8, 444, 32, 444, 1),
                                                      (128, 6, 296, 48, 296, 1), (64, 6, 592, 48, 592, 1)):
            nbytes = tiles * kbs * box * 128
            assert nbytes <= buf.numel()
            for packed in (0, 1):
                def fn():
                    rc = L.atlas_probe_tma_stream(buf.data_ptr(), buf.numel(), tiles, kbs, box, stages, packed, ctas, pieces, K._status_ptr[0],
                                                  sink.data_ptr(), K._stream())
                    assert rc == 0, rc
                ms = T.time(fn, iters=5)
                add(f"tma_stream slot={box}x128B in {pieces} copies, stages={stages} ctas={ctas} k_slices={kbs} layout={'packed' if packed else 'weight'}",
                    ms, bytes_=nbytes, note=f"{stages * box * 128 // 1024} KB in flight per CTA")
        # per-thread 16-byte asynchronous copies instead of the copy engine: 4 KB chunks (a K + V page of one kv head), four
        # warps per CTA, several CTAs per SM
        L.atlas_probe_cpasync_stream.argtypes = [C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        for ctas, chunk, depth in ((148 * 4, 4096, 2), (148 * 4, 4096, 3), (148 * 4, 4096, 4), (148 * 6, 4096, 2), (148 * 8, 2048, 4),
                                   (148 * 4, 2048, 6), (148 * 2, 8192, 4), (148 * 4, 8192, 2)):
            per_warp = min(256, buf.numel() // (ctas * 4 * chunk))
            nbytes = ctas * 4 * per_warp * chunk
            def fn():
                rc = L.atlas_probe_cpasync_stream(buf.data_ptr(), buf.numel(), ctas, chunk, depth, per_warp, sink.data_ptr(), K._stream())
                assert rc == 0, rc
            ms = T.time(fn, iters=5)
            add(f"cp.async stream chunk={chunk}B depth={depth} ctas={ctas} ({ctas // 148} per SM) chunks_per_warp={per_warp}", ms,
                bytes_=nbytes, note=f"{4 * depth * chunk // 1024} KB of ring per CTA")
        assert K.check_status() == 0
        return rows

    if only and only.startswith("timeline"):
        # Where the time goes INSIDE one decode-size FP8 GEMM launch: every CTA stamps its phases (GemmParams::timeline),
        # one traced launch per shape after warm-up, cold L2.  only = "timeline" or "timeline:<M>,<M>,..."
        import ctypes as C
        import statistics as st
        ms_list = [int(v) for v in only.split(":")[1].split(",")] if ":" in only else [1, decode_batch]
        L = K.lib()
        L.atlas_gemm_set_timeline.argtypes = [C.c_void_p]
        L.atlas_gemm_set_timeline.restype = None
        tbuf = torch.zeros(160, 32, dtype=torch.int64, device=dev)
        phases = [("prologue", 1, 2), ("wait_prev_kernel", 2, 3), ("first_issue", 3, 4), ("first_tile_lands", 4, 5),
                  ("mma_first_to_last", 5, 6), ("last_fold_after_last_mma", 6, 8),
                  ("splitk_exchange", 8, 9), ("final_epilogue", 9, 10), ("teardown", 10, 11), ("whole_cta", 1, 11),
                  ("cluster_send", 9, 19), ("cluster_barrier", 19, 20), ("cluster_sum", 20, 21), ("cluster_store", 21, 10)]
        for M in ms_list:
            x = torch.randn(M, max(H, I), device=dev).bfloat16()
            for name, N, Kd in gemms:
                wq, ws = Q.quantize_fp8_block(torch.randn(N, Kd, device=dev) * 0.02)
                xq, xs = K.quant_fp8(x[:, :Kd].contiguous())
                res = torch.randn(M, N, device=dev).bfloat16()
                nw = torch.ones(N, device=dev).bfloat16()
                mode = 1 if name == "gate_up" else (2 if name in ("o", "down") else 0)
                fn = (lambda: K.gemm_fp8_fused(xq, xs, wq, ws, mode=mode, residual=res if mode == 2 else None,
                                               norm_w=nw if mode == 2 else None))
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                T.flush.fill_(1)
                tbuf.zero_()
                torch.cuda.synchronize()
                L.atlas_gemm_set_timeline(tbuf.data_ptr())
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                L.atlas_gemm_set_timeline(None)
                t = tbuf.cpu()
                live = t[t[:, 0] != 0]
                mhz = [float(r[11] - r[1]) / max(1.0, float(r[12] - r[0])) * 1e3 for r in live if r[12] > r[0]]
                clk = st.median(mhz) if mhz else 1900.0
                us = lambda cyc: cyc / clk
                rec = {"kernel": f"timeline {name} M={M} N={N} K={Kd} mode={mode}", "ctas": int(live.shape[0]),
                       "event_us": round(e0.elapsed_time(e1) * 1e3, 1),
                       "span_us": round(float(live[:, 12].max() - live[:, 0].min()) / 1e3, 1),
                       "entry_skew_us_max": round(float(live[:, 0].max() - live[:, 0].min()) / 1e3, 1), "sm_mhz": round(clk)}
                for label, a, b in phases:
                    d = [us(float(r[b] - r[a])) for r in live if r[a] and r[b]]
                    if d:
                        rec[label] = [round(st.median(d), 2), round(max(d), 2)]
                rec["note"] = "phase values are [median, max] microseconds over the CTAs"
                rows.append(rec)
                print(json.dumps(rec), flush=True)
        return rows

    if only and "sweep" in only:
        # tile / split-K sweep for the decode-size FP8 GEMMs
        for M in (decode_batch,):
            x = torch.randn(M, max(H, I), device=dev).bfloat16()
            for name, N, Kd in gemms:
                w = torch.randn(N, Kd, device=dev) * 0.02
                wq, ws = Q.quantize_fp8_block(w)
                del w
                xq, xs = K.quant_fp8(x[:, :Kd].contiguous())
                out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
                for bn in (64, 128):
                    for sp in (1, 2, 4, 8):
                        K._FORCE_BLOCK_N, K._FORCE_SPLITS = bn, sp
                        ms = T.time(lambda: K.gemm_fp8_block(xq, xs, wq, ws, out=out), iters=5)
                        add(f"sweep gemm_fp8 {name} M={M} N={N} K={Kd} bn={bn} splits={sp}", ms,
                            bytes_=N * Kd + M * Kd + 2 * M * N)
                K._FORCE_BLOCK_N = K._FORCE_SPLITS = 0
                del wq, ws

    if not only or "elt" in only:
        for M in (decode_batch, chunk):
            x = torch.randn(M, H, device=dev).bfloat16()
            r = torch.randn(M, H, device=dev).bfloat16()
            wn = torch.ones(H, device=dev).bfloat16()
            ms = T.time(lambda: K.rmsnorm(x, wn, 1e-5, r, False, quant=True))
            add(f"residual_rmsnorm_quant T={M} H={H}", ms, bytes_=M * H * (2 + 2 + 2 + 1))
            gu = torch.randn(M, 2 * I, device=dev).bfloat16()
            ms = T.time(lambda: K.silu_mul(gu, quant=True))
            add(f"silu_mul_quant T={M} I={I}", ms, bytes_=M * I * (4 + 1))

    if not only or "attn" in only:
        bs = 16
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        B = decode_batch
        nblk = (ctx + bs - 1) // bs
        nb = B * nblk + 8
        kc, vc = K.alloc_kv_cache(nb, bs, Hkv, D, torch.float8_e4m3fn, dev)
        kc.copy_((torch.randn(nb, bs, Hkv, D, device=dev) * 0.5).to(torch.float8_e4m3fn))
        vc.copy_((torch.randn(nb, bs, Hkv, D, device=dev) * 0.5).to(torch.float8_e4m3fn))
        perm = torch.randperm(nb - 8).tolist()
        tables = [perm[i * nblk:(i + 1) * nblk] for i in range(B)]
        fb = ForwardBatch.build([[0]] * B, [ctx - 1] * B, tables, bs, device=dev)
        q = (torch.randn(B, Hq, D, device=dev) * 0.5).bfloat16()
        ms = T.time(lambda: K.paged_attention(q, kc, vc, fb, D ** -0.5, 1.0, 1.0, None))
        add(f"attn_decode B={B} ctx={ctx} Hq={Hq} Hkv={Hkv} D={D}", ms, bytes_=2 * B * ctx * Hkv * D,
            flops=4 * B * ctx * Hq * D)
        # rope + kv write at decode
        qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
        rope = ref.build_rope_cache(D, 4096, 5e5, None, dev)
        qv = qkv[:, :Hq * D].view(B, Hq, D)
        kv_ = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, Hkv, D)
        vv = qkv[:, (Hq + Hkv) * D:].view(B, Hkv, D)
        ms = T.time(lambda: K.qk_norm_rope_kv_write(qv, kv_, vv, fb.positions, rope, D, kc, vc, fb.slot_mapping, 1.0, 1.0,
                                                    None, None, 1e-6, False))
        add(f"rope_kv_write T={B}", ms, bytes_=B * (Hq + 2 * Hkv) * D * 2 * 2)
        # prefill: chunk tokens as sequences of 1024
        n_seq = max(1, chunk // 1024)
        L = 1024
        nblk = L // bs
        tables = [perm[i * nblk:(i + 1) * nblk] for i in range(n_seq)]
        fbp = ForwardBatch.build([[0] * L] * n_seq, [0] * n_seq, tables, bs, device=dev)
        qp = (torch.randn(n_seq * L, Hq, D, device=dev) * 0.5).bfloat16()
        ms = T.time(lambda: K.paged_attention(qp, kc, vc, fbp, D ** -0.5, 1.0, 1.0, None), iters=5)
        add(f"attn_prefill seqs={n_seq} len={L} Hq={Hq} Hkv={Hkv} D={D}", ms, flops=4 * n_seq * Hq * D * L * L // 2)
        qkvp = torch.randn(n_seq * L, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
        qv = qkvp[:, :Hq * D].view(-1, Hq, D)
        kv_ = qkvp[:, Hq * D:(Hq + Hkv) * D].view(-1, Hkv, D)
        vv = qkvp[:, (Hq + Hkv) * D:].view(-1, Hkv, D)
        ms = T.time(lambda: K.qk_norm_rope_kv_write(qv, kv_, vv, fbp.positions, rope, D, kc, vc, fbp.slot_mapping, 1.0, 1.0,
                                                    None, None, 1e-6, False))
        add(f"rope_kv_write T={n_seq * L}", ms, bytes_=n_seq * L * (Hq + 2 * Hkv) * D * 2 * 2)

    if only and "gdn" in only:
        # Gated-DeltaNet prefill (Qwen3-Next geometry): conv + chunked scan + state write, one layer
        from atlas_b200.layers import ParallelCtx
        from atlas_b200.layers.gdn import GatedDeltaNet
        from atlas_b200.ops import cuda_gdn
        gcfg = PRESETS["qwen3-next-80b"]()
        layer = GatedDeltaNet(gcfg, 0, ParallelCtx(), "dense")
        layer.conv_w = (torch.randn(layer.conv_dim, layer.W, device=dev) * 0.2).bfloat16()
        layer.dt_bias = torch.rand(layer.hv, device=dev)
        layer.A_log = torch.log(torch.rand(layer.hv, device=dev) * 15 + 1)
        T.use_graph = False
        for n_seq, L in ((8, 1024), (1, chunk)):
            st_ = layer.alloc_state(n_seq + 1, dev, torch.bfloat16)
            mixed = torch.randn(n_seq * L, layer.conv_dim, device=dev).bfloat16()
            ga = torch.randn(n_seq * L, layer.hv, device=dev).bfloat16()
            gb = torch.randn(n_seq * L, layer.hv, device=dev).bfloat16()
            fbg = ForwardBatch.build([[0] * L] * n_seq, [0] * n_seq, [list(range((L + 15) // 16))] * n_seq, 16, device=dev,
                                     state_slots=list(range(n_seq)), has_state=[False] * n_seq)
            for chunked in (True, False):
                cuda_gdn.USE_CHUNKED = chunked
                ms = T.time(lambda: K.gdn_forward(layer, mixed, ga, gb, fbg, st_, commit=True), iters=3)
                add(f"gdn_prefill Hk={layer.hk} Hv={layer.hv} D=128 seqs={n_seq} L={L} {'chunked' if chunked else 'sequential'}", ms,
                    bytes_=n_seq * L * (layer.conv_dim * 2 * 2 + layer.hv * 128 * 2))
        cuda_gdn.USE_CHUNKED = True
        T.use_graph = True

    if only and "moe" in only:
        # one MoE FFN (Qwen3-30B-A3B geometry, NVFP4 experts): route + align + gather + grouped GEMMs + combine
        from atlas_b200.layers.moe import ExpertWeights
        E, Hm, Im, topk = 128, 2048, 768, 8
        exw = ExpertWeights.from_dense((torch.randn(E, 2 * Im, Hm, device=dev) * 0.05).bfloat16(),
                                       (torch.randn(E, Hm, Im, device=dev) * 0.05).bfloat16(), "nvfp4")
        T.use_graph = False
        for M in (decode_batch, chunk):
            xm = torch.randn(M, Hm, device=dev).bfloat16()
            tw, ti = ref.moe_route(torch.randn(M, E, device=dev), topk, True)
            tw, ti = tw.contiguous(), ti.contiguous()
            ms = T.time(lambda: K.moe_forward(xm, tw, ti, exw, 0, None, "allreduce"), iters=3)
            wbytes = E * 3 * Im * Hm * 0.5625
            add(f"moe_ffn nvfp4 T={M} E={E} top{topk} H={Hm} I={Im}", ms, bytes_=wbytes, flops=2 * M * topk * 3 * Im * Hm)
        T.use_graph = True

    if not only or "sample" in only:
        lg = torch.randn(decode_batch, cfg.vocab_size, device=dev).bfloat16()
        ms = T.time(lambda: K.argmax(lg))
        add(f"argmax B={decode_batch} V={cfg.vocab_size}", ms, bytes_=2 * decode_batch * cfg.vocab_size)
    st = K.check_status()
    if st:
        print(f"device status word {st:#x}", file=sys.stderr)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--chunk", type=int, default=8192)
    ap.add_argument("--only", default=None)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    rows = run(a.model, a.batch, a.ctx, a.chunk, a.only)
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"peaks": load_peaks(), "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
