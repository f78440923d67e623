"""Lag-one decode pipeline: while the device runs decode step ``N + 1`` the host reads back and applies the tokens of
step ``N``.

A plain decode step does not need the VALUES of the tokens sampled one step earlier on the host: positions, cache slots
and block tables follow from the sequence lengths alone, and the token ids can be fed from the previous step's
device-side sampling result.  The pipeline therefore launches step ``N + 1`` (metadata from pinned host buffers,
input ids copied device to device, CUDA-graph replay, greedy sampling, asynchronous read-back) before it waits for step
``N``.  Stop conditions are evaluated one step late: when a sequence turns out to have finished at step ``N`` its row
in step ``N + 1`` was computed for nothing and is dropped (the cache slot it wrote lies past the sequence's computed
length, in a block that is never published to the prefix cache).

The pipeline only runs while the engine is in its simplest state and hands control back to the general step loop
otherwise: every running sequence is a plain greedy decode (no grammar, logit processors, penalties, log-probs, drafts
or adapters), nothing is waiting, prefilling or swapped, a captured decode graph of the right size exists, and no
multi-process control plane is attached (symmetric tensor-parallel ranks run the same pipeline in lock step because
every decision here is a function of replicated host state).

Reference parity: the reference overlaps host scheduling with device work in its scheduler's decode loop
(``crates/spark-server/src/scheduler/decode_loop.rs``: next-step upload while the current step's tokens are in flight).
"""
from __future__ import annotations

import time
from collections import deque
from typing import Deque, List, Optional

import numpy as np
import torch

from .sched.sequence import ScheduledSeq, SchedulerOutput, SeqStatus

_DEPTH = 2            # steps in flight: one executing, one whose results are being applied
_SETS = 3             # rotating pinned staging sets (a set is reused only after the step that read it has retired)


class DecodePipeline:
    def __init__(self, engine):
        self.eng = engine
        self.active = False
        self.stop = False
        self.seqs: list = []
        self.inflight: Deque[tuple] = deque()
        self.dev_ids: Optional[torch.Tensor] = None
        self.launches = 0
        self._pins: dict = {}
        self._last_retire = 0.0
        self.steps = 0                       # retired pipeline steps (for tests / stats)

    # ------------------------------------------------------------------ eligibility
    def _simple(self, seq) -> bool:
        return (seq.status == SeqStatus.RUNNING and not seq.finished and seq.num_tokens == seq.num_computed + 1
                and not seq.drafts and not seq.adapter_slot and seq.grammar is None and not seq.logits_processors
                and not getattr(seq, "needs_full_logits", False) and getattr(seq, "mm", None) is None)

    def _quiet(self) -> bool:
        s = self.eng.scheduler
        return not s.waiting and not s.prefilling and not s.swapped and not s.finished_queue

    def _graph(self, n: int):
        from .runner import _pad_batch
        g = self.eng.runner.graphs.get(_pad_batch(n))
        return g if (g is not None and g.graph is not None) else None

    def _can_start(self) -> bool:
        eng = self.eng
        run = eng.scheduler.running
        if not run or not self._quiet() or eng.host_tier is not None and eng.scheduler.swapped:
            return False
        if len(run) > max(eng.runner.graph_batch_sizes()) or self._graph(len(run)) is None:
            return False
        if not all(self._simple(s) for s in run) or not eng.sampler.fast_greedy(run):
            return False
        return all(s.sampling.max_tokens - s.num_output_tokens >= 2 for s in run)

    def _can_launch(self) -> bool:
        if not self.active or self.stop or len(self.inflight) >= _DEPTH or not self._quiet():
            return False
        eng, sched = self.eng, self.eng.scheduler
        run = sched.running
        if len(run) != len(self.seqs) or any(a is not b for a, b in zip(run, self.seqs)):
            return False
        n = len(self.inflight)
        now = time.monotonic()
        for s in self.seqs:
            if s.finished or s.status != SeqStatus.RUNNING:
                return False
            if s.num_output_tokens + n >= s.sampling.max_tokens or s.num_tokens + n >= eng.cfg.max_seq_len:
                return False
            if s.deadline is not None and now > s.deadline:
                return False
        return all(sched._ensure_blocks(s, s.num_computed + n + 1) for s in self.seqs)

    # ------------------------------------------------------------------ staging
    def _pin(self, name: str, shape, dtype) -> torch.Tensor:
        key = (name, self.launches % _SETS)
        t = self._pins.get(key)
        if t is None or t.shape != tuple(shape) or t.dtype != dtype:
            t = self._pins[key] = torch.zeros(shape, dtype=dtype).pin_memory()      # zeros: padding rows keep valid block ids
        return t

    # ------------------------------------------------------------------ launch / retire
    def _launch(self) -> None:
        eng = self.eng
        r = eng.runner
        seqs = self.seqs
        B, n = len(seqs), len(self.inflight)
        g = self._graph(B)
        P, bs = g.P, r.bs
        starts = np.fromiter((s.num_computed + n for s in seqs), dtype=np.int64, count=B)
        mb = g.tables.shape[1]
        table = self._pin("tables", (P, mb), torch.int32)
        tnp = table.numpy()
        for i, s in enumerate(seqs):
            t = r._blocks_np(s)
            tnp[i, :t.shape[0]] = t
        pos = self._pin("pos", (P,), torch.int32)
        slots = self._pin("slots", (P,), torch.int32)
        sl = self._pin("sl", (P,), torch.int32)
        pnp, snp, lnp = pos.numpy(), slots.numpy(), sl.numpy()
        pnp[:B] = starts
        snp[:B] = tnp[np.arange(B), starts // bs].astype(np.int64) * bs + starts % bs
        lnp[:B] = starts + 1
        pnp[B:], snp[B:], lnp[B:] = 0, -1, 1
        ev0 = torch.cuda.Event(enable_timing=True)
        ev0.record()
        if n == 0:
            ids = self._pin("ids", (P,), torch.int64)
            inp = ids.numpy()
            inp[:B] = [s.token_at(int(p)) for s, p in zip(seqs, starts)]
            inp[B:] = 0
            g.ids.copy_(ids, non_blocking=True)
            r.h2d_bytes += P * 8
        else:
            g.ids[:B].copy_(self.dev_ids, non_blocking=True)          # last step's samples, device to device
        g.pos.copy_(pos, non_blocking=True)
        g.slots.copy_(slots, non_blocking=True)
        g.seq_lens.copy_(sl, non_blocking=True)
        g.tables.copy_(table, non_blocking=True)
        r.h2d_bytes += P * 12 + P * mb * 4
        g.graph.replay()
        r.graph_replays += 1
        hidden = g.out[:B]
        if getattr(eng.model, "vocab_parallel", False):
            toks = eng.model.greedy_tokens(hidden)
        else:
            from . import ops
            toks = ops.argmax(eng.model.compute_logits(hidden))
        toks = toks.to(torch.int64)
        self.dev_ids = toks
        out = self._pin("out", (P,), torch.int64)
        out[:B].copy_(toks, non_blocking=True)
        ev1 = torch.cuda.Event(enable_timing=True)
        ev1.record()
        self.inflight.append((ev0, ev1, out, starts))
        self.launches += 1

    def _retire(self) -> List:
        eng, sched = self.eng, self.eng.scheduler
        ev0, ev1, out, starts = self.inflight.popleft()
        ev1.synchronize()
        B = len(self.seqs)
        toks = out[:B].tolist()
        if eng.time_device:
            ms = ev0.elapsed_time(ev1)
            eng.device_time_ms += ms
            d = eng.device_phase_ms.setdefault("decode", [0.0, 0])
            d[0] += ms
            d[1] += 1
        now = time.monotonic()
        results, items = [], []
        for i, seq in enumerate(self.seqs):
            if seq.finished or seq.status != SeqStatus.RUNNING:
                continue                                   # finished one step earlier (or aborted): this row is dropped
            it = ScheduledSeq(seq, int(starts[i]), 1, True, True)
            items.append(it)
            sched.on_chunk_computed(it)
            kept = eng._append_tokens(seq, [int(toks[i])], now, None)
            results.append(eng._make_output(seq, kept))
            if seq.finished:
                eng._seqs.pop(seq.request_id, None)
                eng._stop_checkers.pop(seq.request_id, None)
                self.stop = True
        dt = now - self._last_retire if self._last_retire else 0.0
        self._last_retire = now
        eng.stats.on_step(dt, SchedulerOutput(items=items), sum(len(r.new_tokens) for r in results))
        self.steps += 1
        return results

    # ------------------------------------------------------------------ one engine tick
    def step(self) -> Optional[List]:
        """Results of one tick, or None when the pipeline is not running (the caller takes the general path)."""
        if not self.active:
            if not self._can_start():
                return None
            self.active, self.stop = True, False
            self.seqs = list(self.eng.scheduler.running)
            self.dev_ids = None
            self._last_retire = time.monotonic()
        launched = False
        if self._can_launch():
            self._launch()
            launched = True
        results: List = []
        if self.inflight and (len(self.inflight) >= _DEPTH or not launched):
            results = self._retire()
        if not self.inflight and not launched:
            self.active = False
            self.seqs = []
            if not results:
                return None
        return results
