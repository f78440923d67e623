"""LLMEngine: the public, in-process API of the inference engine.

``add_request`` queues a tokenised prompt, ``step`` runs one continuous-batching iteration (schedule ->
forward -> sample -> emit) and returns the requests that produced tokens, ``generate`` drives steps
until a list of prompts has finished.  The HTTP server wraps an engine in a single scheduler thread
that owns the CUDA context (reference: ``crates/spark-server/src/scheduler/mod.rs:262`` ``run``,
``crates/spark-model/src/engine.rs:26`` ``generate``).
"""
from __future__ import annotations

import itertools
import os
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Hashable, List, Optional, Sequence as Seq

import torch

from .config import EngineConfig, ModelConfig
from .kv import BlockPool, RadixCache, SlotPool
from .models import CacheStore, DecoderLM, ForwardBatch
from .runner import ModelRunner
from .sampling import Sampler, SamplingParams, SamplerOutput
from .sched import FinishReason, ScheduledSeq, Scheduler, SchedulerOutput, SeqStatus, Sequence
from .sched.spec import SpecController
from .utils.metrics import EngineStats
from .utils.trace import phase


@dataclass
class RequestOutput:
    request_id: str
    new_tokens: List[int]
    output_tokens: List[int]
    finished: bool
    finish_reason: Optional[str] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0
    ttft_s: Optional[float] = None
    decode_time_s: Optional[float] = None
    logprobs: Optional[List[Any]] = None
    accepted_prediction_tokens: int = 0


class RequestRejected(ValueError):
    pass


class LLMEngine:
    def __init__(self, model: DecoderLM, cfg: Optional[EngineConfig] = None):
        self.model = model
        self.cfg = cfg or EngineConfig()
        self.mcfg: ModelConfig = model.cfg
        dev = model.device
        self.hybrid = self.mcfg.family == "hybrid" and len(model.gdn_layers()) > 0
        self.kv_dtype = self._resolve_kv_dtype()
        num_blocks = self.cfg.num_kv_blocks or self._profile_num_blocks()
        n_active = self.cfg.max_num_seqs if self.hybrid else 0
        n_snap = self.cfg.ssm_cache_slots if (self.hybrid and self.cfg.enable_prefix_caching) else 0
        self.cache: CacheStore = model.alloc_cache(num_blocks, self.cfg.block_size, self.kv_dtype, n_active + n_snap,
                                                   high_precision_layers=self.cfg.kv_high_precision_layers)
        if os.environ.get("ATLAS_NATIVE_RUNTIME", "0") not in ("0", "", "false"):
            from .runtime_native import NativeBlockPool          # C++ pool, same interface
            self.pool = NativeBlockPool(num_blocks, self.cfg.block_size)
        else:
            self.pool = BlockPool(num_blocks, self.cfg.block_size)
        self.state_pool = SlotPool(n_active) if self.hybrid else None
        self.snapshot_base = n_active
        self.radix = RadixCache(self.pool, snapshot_slots=n_snap) if self.cfg.enable_prefix_caching else None
        self.host_tier = None
        if self.cfg.swap_space_gb > 0:
            from .kv.host_tier import HostKVTier
            per_block = max(1, model.kv_bytes_per_block(self.cfg.block_size, self.kv_dtype, self.cfg.kv_high_precision_layers))
            n_host = int(self.cfg.swap_space_gb * (1 << 30)) // per_block
            if n_host > 0:
                self.host_tier = HostKVTier(self.cache, n_host, self.cfg.max_num_seqs if self.hybrid else 0,
                                            disk_gb=self.cfg.disk_swap_gb, disk_dir=self.cfg.disk_swap_path)
        self.selector = None
        if self.cfg.sparse_attention_blocks > 0:
            from .kv.sparse_select import BlockSelector
            from .layers import Attention
            self.selector = BlockSelector(num_blocks, self.cfg.block_size, self.cfg.sparse_attention_blocks)
            for l in model.layers:
                if l.kind == "attention" and type(l.mixer) is Attention:
                    l.mixer.selector = self.selector
        self.scheduler = Scheduler(self.cfg, self.pool, self.radix, self.state_pool, self.hybrid, host_tier=self.host_tier)
        self.sampler = Sampler(self.mcfg.vocab_size, self.mcfg.eos_ids())
        # largest step this engine can build: sizes the sequence-parallel peer-memory area once
        model.sp_capacity_hint = self.cfg.max_prefill_tokens + self.cfg.max_num_seqs * (1 + max(0, self.cfg.num_drafts))
        self.runner = ModelRunner(model, self.cache, self.cfg)
        self.spec = SpecController(self, self.cfg) if (self.cfg.speculative and model.mtp is not None
                                                         and self.cfg.num_drafts > 0) else None
        if self.spec is not None and 0 < self.cfg.mtp_draft_vocab < self.mcfg.vocab_size:
            from .utils.vocab_rank import load_ranked_ids, select_rows
            ranked = None if self.cfg.mtp_vocab_rank in ("", "id") else load_ranked_ids(self.cfg.mtp_vocab_rank)
            model.build_draft_head(select_rows(self.cfg.mtp_draft_vocab, self.mcfg.vocab_size, ranked, self.mcfg.eos_ids()),
                                   "fp8_block" if model.device.type == "cuda" else "dense")
        if self.spec is None and self.cfg.speculative and getattr(model, "dflash", None) is not None and self.cfg.num_drafts > 0:
            from .sched.spec import DFlashSpecController
            model.dflash.alloc_cache(num_blocks, self.cfg.block_size)
            model.dflash.finalize(self.cfg.max_seq_len + self.cfg.num_drafts + 8)
            model.capture_layers = tuple(model.dflash.dcfg.target_layer_ids)
            model.graph_safe = False            # the captured states must be this step's tensors, not a graph's
            self.spec = DFlashSpecController(self, self.cfg)
        if self.spec is None and self.cfg.self_speculative and self.cfg.num_drafts > 0:
            from .sched.spec import SelfSpecController
            if SelfSpecController.supported(model):
                self.spec = SelfSpecController(self, self.cfg)
        if self.spec is None and self.cfg.ngram_speculative and self.cfg.num_drafts > 0:
            from .sched.spec import NgramSpecController
            self.spec = NgramSpecController(self, self.cfg)     # draft-model-free: works for every architecture
        self.stats = EngineStats()
        self.control = None               # parallel.worker.StepControl when several processes serve one model
        self._eos_set = frozenset(self.mcfg.eos_ids())
        self.time_device = False          # accumulate CUDA-event time of each step's GPU work
        self._pipe = None                 # pipeline.DecodePipeline (lag-one decode loop), created on first use
        self.device_phase_ms: Dict[str, list] = {}     # phase -> [ms, steps] (steps with any multi-token item count as prefill)
        self.device_time_ms = 0.0
        self._seqs: Dict[str, Sequence] = {}
        self._ids = itertools.count()
        self._stop_checkers: Dict[str, Callable[[Sequence], bool]] = {}

    # ------------------------------------------------------------------ sizing
    def _resolve_kv_dtype(self) -> torch.dtype:
        want = self.cfg.kv_cache_dtype
        if want == "auto":
            want = self.mcfg.quant.kv_cache_dtype
        if want == "nvfp4":
            # packed e2m1 + e4m3 block scales: 0.56 bytes per element.  The cache writer and the attention kernel exist for
            # head_dim 128 with full rotary width on the GPU; anything else keeps the FP8 cache.
            ok = (self.model.device.type == "cuda" and self.mcfg.head_dim == 128 and self.mcfg.rotary_dim == 128
                  and self.mcfg.kv_lora_rank == 0 and self.cfg.block_size % 16 == 0 and not self.cfg.sparse_attention_blocks)
            if ok:
                from .models.decoder import KV_NVFP4
                return KV_NVFP4
            want = "fp8"
        if want == "turbo8":
            # Hadamard-rotated heads in an FP8 cache: same bytes and the same attention kernels as "fp8"; a model the
            # rotation does not cover keeps the plain FP8 cache
            self.model.set_kv_rotation(True)
            want = "fp8"
        if want == "bf16":
            return torch.bfloat16           # GPU: the general mma.sync attention kernel on a 16-bit cache
        if want == "fp8" or (want == "auto" and self.model.device.type == "cuda"):
            return torch.float8_e4m3fn      # default on a GPU: the bulk-copy decode and tcgen05 prefill kernels
        return self.model.dtype

    def _profile_num_blocks(self) -> int:
        per_block = max(1, self.model.kv_bytes_per_block(self.cfg.block_size, self.kv_dtype, self.cfg.kv_high_precision_layers))
        if self.model.device.type == "cuda":
            free, total = torch.cuda.mem_get_info(self.model.device)
            budget = int(total * self.cfg.gpu_memory_utilization) - (total - free)
            # keep headroom for activations of the largest prefill chunk and the graph pools
            budget -= self.runner_activation_reserve()
            n = max(16, budget // per_block)
        else:
            n = 4096
        cap = (self.cfg.max_seq_len // self.cfg.block_size + 1) * self.cfg.max_num_seqs
        return int(min(n, cap))

    def runner_activation_reserve(self) -> int:
        c = self.mcfg
        widest = max(c.q_size + 2 * c.kv_size, 2 * max(c.intermediate_size, c.moe_intermediate_size * max(1, c.num_experts_per_tok)),
                     c.hidden_size)
        tp = max(1, self.model.pctx.tp_size)
        act = self.cfg.max_prefill_tokens * (widest // tp + 4 * c.hidden_size) * 2 * 3
        logits = self.cfg.max_num_seqs * c.vocab_size * 6
        return int(act + logits + (2 << 30))

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_tokens: Seq[int], sampling: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, namespace: Hashable = 0, priority: int = 0,
                    timeout_s: Optional[float] = None, grammar: Any = None,
                    logits_processors: Optional[List[Callable]] = None, disable_spec: bool = False,
                    stop_checker: Optional[Callable[[Sequence], bool]] = None, adapter_slot: int = 0,
                    needs_full_logits: bool = False, images: Optional[List[tuple]] = None) -> str:
        """``needs_full_logits``: set on follower ranks for a request whose leader-side sampling needs the whole
        logits row (grammar mask, logit processors), so that every rank takes the same path to the logits.
        ``images``: ``(patches, (t, h, w))`` pairs (see ``models.vision.patchify``) for a prompt that already carries one
        run of image placeholder tokens per image, ``h * w / merge^2`` tokens long."""
        sampling = sampling or SamplingParams()
        sampling.validate()
        rid = request_id or f"req-{next(self._ids)}"
        prompt = [int(t) for t in prompt_tokens]
        if not prompt:
            raise RequestRejected("empty prompt")
        if any(t < 0 or t >= self.mcfg.vocab_size for t in prompt):
            raise RequestRejected("token id out of range")
        total = len(prompt) + sampling.max_tokens
        if len(prompt) >= self.cfg.max_seq_len:
            raise RequestRejected(f"prompt of {len(prompt)} tokens exceeds max_seq_len {self.cfg.max_seq_len}")
        if total > self.cfg.max_seq_len:
            sampling.max_tokens = self.cfg.max_seq_len - len(prompt)
        if self.pool.blocks_for_tokens(len(prompt) + 1) > self.pool.num_blocks:
            raise RequestRejected("prompt does not fit in the KV cache")
        t_out = timeout_s if timeout_s is not None else (self.cfg.request_timeout_s or None)
        seq = Sequence(rid, prompt, sampling, namespace=(adapter_slot, namespace), priority=priority,
                       deadline=(time.monotonic() + t_out) if t_out else None, grammar=grammar,
                       logits_processors=list(logits_processors or []), disable_spec=disable_spec,
                       adapter_slot=adapter_slot)
        seq.needs_full_logits = bool(needs_full_logits or grammar is not None or logits_processors)
        if images:
            if self.model.vision is None:
                raise RequestRejected("this model has no vision tower")
            from .models.vision import prepare
            try:
                seq.mm = prepare(self.model.vision, prompt, self.mcfg.image_token_id, images)
            except ValueError as exc:
                raise RequestRejected(str(exc))
            seq.namespace = ("mm", rid)           # placeholder ids say nothing about the pixels: no prefix sharing
        self._seqs[rid] = seq
        if stop_checker is not None:
            self._stop_checkers[rid] = stop_checker
        self.scheduler.add(seq)
        self.stats.requests_total += 1
        return rid

    def abort(self, request_id: str) -> bool:
        s = self.scheduler.abort(request_id)
        self._seqs.pop(request_id, None)
        self._stop_checkers.pop(request_id, None)
        return s is not None

    def load_adapter(self, name: str, path: str) -> int:
        """Read a PEFT adapter directory and make it resident under ``name``; returns its slot (the value requests pass
        as ``adapter_slot``).  On a tensor-parallel rank the adapter is cut like the base weights."""
        from .lora import load_adapter
        ad = load_adapter(path, self.model)
        ad.name = name
        return self.model.register_adapter(ad)

    def unload_adapter(self, name: str) -> None:
        if getattr(self.model, "lora", None) is not None:
            self.model.lora.unregister(name)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ one step
    @torch.inference_mode()
    def step(self) -> List[RequestOutput]:
        """One scheduler tick.  With a multi-process ``control`` attached the leader's clock, request events and
        sampling outcome are imposed on the followers (see ``parallel/worker.py``); otherwise everything is local."""
        t0 = time.monotonic()
        sched = self.scheduler
        ctl = self.control
        if ctl is None and self.spec is None and self.cfg.async_decode and self.model.device.type == "cuda":
            if self._pipe is None:
                from .pipeline import DecodePipeline
                self._pipe = DecodePipeline(self)
            piped = self._pipe.step()
            if piped is not None:
                return piped
        follower = ctl is not None and not ctl.is_leader
        now_plan = ctl.begin_step(self) if ctl is not None else None
        with phase("schedule"):
            out = sched.schedule(now=now_plan, expire=ctl is None)
        results: List[RequestOutput] = []
        for s in sched.finished_queue:      # deadline expiries
            results.append(self._make_output(s, []))
            self._seqs.pop(s.request_id, None)
        sched.finished_queue.clear()
        # host-tier traffic of this plan: saves first (a released block may already belong to someone else), then restores
        for host_blocks, records in out.disk_out:
            self.host_tier.spill(host_blocks, records)
        for dev_blocks, host_blocks, state_slot, host_state in out.swap_out:
            self.host_tier.copy_out(dev_blocks, host_blocks, state_slot, host_state)
        for records, host_blocks in out.disk_in:
            self.host_tier.unspill(records, host_blocks)
            self.host_tier.disk.free(records)
        for host_blocks, dev_blocks, host_state, state_slot in out.swap_in:
            self.host_tier.copy_in(host_blocks, dev_blocks, host_state, state_slot)
            self.host_tier.free(host_blocks)
            self.host_tier.free_state(host_state)
        if out.empty:
            if ctl is not None:
                ctl.finish_step(None if follower else _empty_outcome())
            return results
        for snap_slot, seq_slot in out.restored_snapshots:
            self.runner.copy_state(self.snapshot_base + snap_slot, seq_slot)
        use_spec = self.spec is not None and self.spec.active()
        with phase("build_batch"):
            batch = self.runner.build_batch(out, self.snapshot_base)
        ev = None
        if self.time_device and self.model.device.type == "cuda":
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        with phase("forward", tokens=batch.num_tokens if hasattr(batch, "num_tokens") else 0):
            hidden = self.runner.forward(batch)
        # rows that need logits
        rows, row_owner = [], []
        qsl = 0
        for idx, it in enumerate(out.items):
            if it.sample:
                if it.verify_drafts:
                    rows.extend(range(qsl, qsl + it.num_tokens))
                    row_owner.extend([idx] * it.num_tokens)
                else:
                    rows.append(qsl + it.num_tokens - 1)
                    row_owner.append(idx)
            qsl += it.num_tokens
        sampled: Dict[int, List[int]] = {}
        lps: Dict[int, list] = {}
        if rows:
            seqs_rows = [out.items[i].seq for i in row_owner]
            verify = any(out.items[i].verify_drafts for i in set(row_owner))
            # vocab-parallel head and a plain greedy step: exchange one (max, index) pair per row instead of gathering
            # the logits.  The test only reads replicated request state, so every rank decides alike.
            greedy_tp = (getattr(self.model, "vocab_parallel", False) and not verify
                         and self.sampler.fast_greedy(seqs_rows))
            with phase("logits"):
                # every rank: the vocab-parallel gather / exchange is a collective
                logits = self.runner.greedy_tokens(hidden, rows) if greedy_tp else self.runner.logits(hidden, rows)
            self._device_accept = None
            if not follower:
                so = SamplerOutput(logits.tolist()) if greedy_tp else (
                    self.sampler(logits, seqs_rows) if not verify else self._sample_verify_rows(logits, out, row_owner))
                for j, i in enumerate(row_owner):
                    sampled.setdefault(i, []).append(so.tokens[j])
                    if so.logprobs is not None and so.logprobs[j] is not None:
                        lps.setdefault(i, []).append(so.logprobs[j])
        if ev is not None:
            ev[1].record()
            ev[1].synchronize()
            ms = ev[0].elapsed_time(ev[1])
            self.device_time_ms += ms
            kind = "decode" if all(it.num_tokens == 1 for it in out.items) else "prefill"
            d = self.device_phase_ms.setdefault(kind, [0.0, 0])
            d[0] += ms
            d[1] += 1
        now = time.monotonic()
        dt_gate: Optional[float] = None
        if follower:
            outcome = ctl.finish_step(None)
            accepted_rows = self._apply_outcome(out, outcome.records, now)
            dt_gate = outcome.dt
        else:
            with phase("apply"):
                accepted_rows, records = self._apply_sampled(out, sampled, lps, now, results)
            if ctl is not None:
                dt_gate = time.monotonic() - t0
                ctl.finish_step(_make_outcome(records, dt_gate))
        if batch.spec_verify:
            self.model.commit_spec(accepted_rows, self.cache)
            for it in out.items:
                if not it.seq.finished:
                    sched.trim_blocks(it.seq)
        if use_spec:
            self.spec.after_step(out, batch, hidden, sampled, accepted_rows)
        dt = time.monotonic() - t0
        n_new = sum(len(r.new_tokens) for r in results)
        self.stats.on_step(dt, out, n_new)
        if self.spec is not None:
            n_gate = n_new if not follower else sum(len(v[1]) for v in outcome.records.values())
            self.spec.gate.record(batch.spec_verify, dt if dt_gate is None else dt_gate, n_gate)
        return results

    def _apply_sampled(self, out: SchedulerOutput, sampled: Dict[int, List[int]], lps: Dict[int, list], now: float,
                       results: List[RequestOutput]):
        """Authoritative post-processing: draft acceptance, appends, stop conditions.  Returns the rows kept per
        item and the per-item records a follower needs to replay the same state changes."""
        sched = self.scheduler
        accepted_rows: List[int] = []
        records: Dict[int, tuple] = {}
        for idx, it in enumerate(out.items):
            seq = it.seq
            new_tokens: List[int] = []
            if it.verify_drafts:
                targets = sampled[idx]
                dev_acc = getattr(self, "_device_accept", None)
                if dev_acc is not None and idx in dev_acc:
                    n_acc = dev_acc[idx]                    # counted on the device (spec_accept kernel)
                else:
                    n_acc = 0
                    while n_acc < it.verify_drafts and seq.drafts[n_acc] == targets[n_acc]:
                        n_acc += 1
                new_tokens = targets[:n_acc + 1]
                seq.spec_proposed += it.verify_drafts
                seq.spec_accepted += n_acc
                self.stats.spec_proposed += it.verify_drafts
                self.stats.spec_accepted += n_acc
                sched.on_chunk_computed(it, n_acc + 1)
                accepted_rows.append(n_acc + 1)
                seq.drafts = []
            else:
                sched.on_chunk_computed(it)
                accepted_rows.append(it.num_tokens)
                if it.sample:
                    new_tokens = sampled[idx]
            kept: List[int] = []
            if new_tokens:
                kept = self._append_tokens(seq, new_tokens, now, lps.get(idx))
                if seq.status == SeqStatus.PREFILL and not seq.finished:
                    sched.promote(seq)
                results.append(self._make_output(seq, kept))
                if seq.finished:
                    self._seqs.pop(seq.request_id, None)
                    self._stop_checkers.pop(seq.request_id, None)
            records[idx] = (accepted_rows[-1], kept, seq.finish_reason.value if seq.finished else None)
        return accepted_rows, records

    def _apply_outcome(self, out: SchedulerOutput, records: Dict[int, tuple], now: float) -> List[int]:
        """Follower replay of the leader's outcome (no sampling, no stop logic of its own)."""
        sched = self.scheduler
        accepted_rows: List[int] = []
        for idx, it in enumerate(out.items):
            seq = it.seq
            rows_kept, kept, fin = records[idx]
            if it.verify_drafts:
                sched.on_chunk_computed(it, rows_kept)
                seq.drafts = []
            else:
                sched.on_chunk_computed(it)
            accepted_rows.append(rows_kept)
            if kept:
                if seq.first_token_time is None:
                    seq.first_token_time = now
                seq.output_tokens.extend(int(t) for t in kept)
                self.stats.generation_tokens += len(kept)
            if fin is not None:
                sched.finish(seq, FinishReason(fin))
                self._seqs.pop(seq.request_id, None)
            elif kept and seq.status == SeqStatus.PREFILL:
                sched.promote(seq)
        return accepted_rows

    def _sample_verify_rows(self, logits, out: SchedulerOutput, row_owner: List[int]):
        """Sample every verify row with the uniform of the output position it would emit at, so that
        accepted tokens equal what plain decoding would have drawn."""
        from .sampling import SamplerOutput
        seqs, offs = [], []
        seen: Dict[int, int] = {}
        for i in row_owner:
            k = seen.get(i, 0)
            seen[i] = k + 1
            seqs.append(_RowView(out.items[i].seq, k))
        toks, lps = self.sampler.sample_tensor(logits, seqs)
        # draft acceptance on the device: one (draft, target) row per verify item, then a single read-back of the
        # sampled tokens together with the accepted counts
        items = [i for i in dict.fromkeys(row_owner) if out.items[i].verify_drafts]
        kmax = max(out.items[i].verify_drafts for i in items)
        draft = torch.full((len(items), kmax), -1, dtype=torch.int64)
        gather = torch.zeros(len(items), kmax + 1, dtype=torch.int64)
        first_row: Dict[int, int] = {}
        for r, i in enumerate(row_owner):
            first_row.setdefault(i, r)
        for j, i in enumerate(items):
            k = out.items[i].verify_drafts
            draft[j, :k] = torch.tensor(out.items[i].seq.drafts[:k], dtype=torch.int64)
            gather[j, :k + 1] = torch.arange(first_row[i], first_row[i] + k + 1)
        dev = toks.device
        if dev.type == "cuda":
            draft, gather = draft.pin_memory().to(dev, non_blocking=True), gather.pin_memory().to(dev, non_blocking=True)
        from . import ops as _ops
        n_acc = _ops.spec_accept(draft, toks[gather])
        both = torch.cat([toks, n_acc.to(torch.int64)]).tolist()
        self._device_accept = {i: int(both[len(row_owner) + j]) for j, i in enumerate(items)}
        return SamplerOutput(both[:len(row_owner)], lps)

    def _append_tokens(self, seq: Sequence, toks: List[int], now: float, lps: Optional[list]) -> List[int]:
        """Append sampled tokens, stopping at EOS / stop ids / max_tokens.  Returns the tokens kept."""
        p = seq.sampling
        kept: List[int] = []
        eos = _EMPTY if p.ignore_eos else self._eos_set
        stop_ids = p.stop_token_ids if len(p.stop_token_ids) < 4 else set(p.stop_token_ids)
        checker = self._stop_checkers.get(seq.request_id) if self._stop_checkers else None
        for j, t in enumerate(toks):
            if seq.first_token_time is None:
                seq.first_token_time = now
                self.stats.on_first_token(now - seq.arrival)
            seq.output_tokens.append(int(t))
            kept.append(int(t))
            if seq.grammar is not None and hasattr(seq.grammar, "accept"):
                seq.grammar.accept(int(t))
            if lps is not None and j < len(lps):
                seq.logprobs.append(lps[j])
            reason = None
            if seq.num_output_tokens >= p.min_tokens and (t in eos or t in stop_ids):
                reason = FinishReason.STOP
            elif checker is not None and checker(seq):
                reason = FinishReason.STOP
            elif seq.num_output_tokens >= p.max_tokens or seq.num_tokens >= self.cfg.max_seq_len:
                reason = FinishReason.LENGTH
            if reason is not None:
                self.scheduler.finish(seq, reason)
                self.stats.requests_finished += 1
                break
        self.stats.generation_tokens += len(kept)
        return kept

    def _make_output(self, seq: Sequence, new_tokens: List[int]) -> RequestOutput:
        ttft = (seq.first_token_time - seq.arrival) if seq.first_token_time else None
        dec = (seq.finish_time - seq.first_token_time) if (seq.finish_time and seq.first_token_time) else None
        # output_tokens / logprobs are the sequence's own lists (not copies: a copy per step per request is quadratic)
        return RequestOutput(seq.request_id, new_tokens, seq.output_tokens, seq.finished,
                             seq.finish_reason.value if seq.finish_reason else None, len(seq.prompt_tokens),
                             seq.num_cached_tokens, ttft, dec, seq.logprobs if seq.logprobs else None,
                             seq.spec_accepted)

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Seq[Seq[int]], sampling: Optional[SamplingParams] = None,
                 samplings: Optional[Seq[SamplingParams]] = None) -> List[RequestOutput]:
        """Run the prompts to completion; results come back in prompt order."""
        import copy
        ids = []
        for i, p in enumerate(prompts):
            sp = copy.deepcopy(samplings[i] if samplings is not None else (sampling or SamplingParams()))
            ids.append(self.add_request(p, sp))
        done: Dict[str, RequestOutput] = {}
        while self.has_unfinished():
            for r in self.step():
                if r.finished:
                    done[r.request_id] = r
        return [done[i] for i in ids]

    def snapshot(self) -> Dict[str, Any]:
        s = self.scheduler.snapshot()
        s.update(self.stats.as_dict())
        if self.radix is not None:
            st = self.radix.stats
            s.update({"prefix_lookups": st.lookups, "prefix_hits": st.hits, "prefix_hit_tokens": st.hit_tokens,
                      "prefix_nodes": self.radix.num_nodes})
        if self.spec is not None:
            s["spec_mode"] = self.spec.gate.mode
        return s


class _RowView:
    """Presents verify row ``k`` of a sequence to the sampler as if ``k`` more tokens were already out."""

    def __init__(self, seq: Sequence, k: int):
        self._seq, self._k = seq, k

    def __getattr__(self, name):
        return getattr(self._seq, name)

    @property
    def num_output_tokens(self) -> int:
        return self._seq.num_output_tokens + self._k

    @property
    def output_tokens(self) -> List[int]:
        return self._seq.output_tokens + self._seq.drafts[:self._k]


_EMPTY = frozenset()


def _make_outcome(records, dt):
    from .parallel.worker import StepOutcome
    return StepOutcome(records, dt)


def _empty_outcome():
    return _make_outcome({}, 0.0)
