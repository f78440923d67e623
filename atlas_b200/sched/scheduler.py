"""Continuous-batching scheduler: admission, chunked prefill, mixed prefill+decode steps,
prefix-cache reuse, preemption with resume, speculative-row planning.

One call to :meth:`Scheduler.schedule` plans one engine step:

1. every RUNNING sequence gets its decode row (plus its pending draft rows when speculating); if a
   KV block is missing and neither the free list nor prefix-cache eviction can supply it, the most
   recently admitted sequence is preempted (its full blocks are published to the prefix cache first,
   so the resume recomputes little);
2. sequences in PREFILL continue with a chunk, sharing a per-step token budget;
3. WAITING requests are admitted in policy order while sequence slots, the token budget and the KV
   watermark (prompt blocks + ``min(max_tokens, watermark)`` decode headroom) allow.

Reference parity: ``crates/spark-server/src/scheduler/mod.rs:454-1162`` (tick), ``admission.rs``,
``preempt.rs``, ``phase_start_prefills.rs``, ``phase_continue_prefills.rs``, ``scheduling_policy.rs:31``.
"""
from __future__ import annotations

import time
from collections import deque
from typing import Deque, Dict, List, Optional

from ..config import EngineConfig
from ..kv.block_manager import BlockPool, SlotPool
from ..kv.radix_cache import RadixCache
from .policy import SchedulingPolicy, make_policy
from .sequence import FinishReason, ScheduledSeq, SchedulerOutput, SeqStatus, Sequence


class Scheduler:
    def __init__(self, cfg: EngineConfig, pool: BlockPool, radix: Optional[RadixCache] = None,
                 state_pool: Optional[SlotPool] = None, hybrid: bool = False,
                 policy: Optional[SchedulingPolicy] = None, host_tier=None):
        self.cfg, self.pool, self.radix, self.state_pool, self.hybrid = cfg, pool, radix, state_pool, hybrid
        self.host_tier = host_tier                    # kv.host_tier.HostKVTier or None: swap instead of recompute
        self.swapped: Deque[Sequence] = deque()
        self._resumed_now: List[Sequence] = []        # resumed in the current schedule() call: not victims yet
        self.num_swaps = 0
        self.num_spills = 0
        self.bs = pool.block_size
        self.policy = policy or make_policy(cfg.scheduling_policy, cfg.tbt_deadline_ms)
        self.waiting: Deque[Sequence] = deque()
        self.prefilling: List[Sequence] = []
        self.running: List[Sequence] = []
        self.finished_queue: List[Sequence] = []
        self.num_preemptions = 0
        self.snapshot_interval = max(self.bs, (cfg.ssm_checkpoint_interval + self.bs - 1) // self.bs * self.bs)
        self._last_decode_time: Optional[float] = None

    # ------------------------------------------------------------------ queue ops
        self.admission_paused = False       # set by the memory watchdog while free memory is under its soft floor

    def add(self, seq: Sequence) -> None:
        seq.status = SeqStatus.WAITING
        self.waiting.append(seq)

    def abort(self, request_id: str, reason: FinishReason = FinishReason.ABORT) -> Optional[Sequence]:
        for q in (self.waiting, self.prefilling, self.running, self.swapped):
            for s in list(q):
                if s.request_id == request_id:
                    q.remove(s)
                    self._release(s, publish=False)
                    s.status, s.finish_reason, s.finish_time = SeqStatus.FINISHED, reason, time.monotonic()
                    return s
        return None

    @property
    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.prefilling) + len(self.running) + len(self.swapped)

    def has_work(self) -> bool:
        return self.num_unfinished > 0

    # ------------------------------------------------------------------ block helpers
    def _reclaim(self, need: int) -> bool:
        """Make ``need`` blocks available, evicting prefix-cache leaves if the free list is short."""
        short = need - self.pool.num_free
        if short > 0 and self.radix is not None:
            self.radix.evict(short)
        return self.pool.num_free >= need

    def _ensure_blocks(self, seq: Sequence, upto_tokens: int) -> bool:
        need = self.pool.blocks_for_tokens(upto_tokens) - len(seq.blocks)
        if need <= 0:
            return True
        if not self._reclaim(need):
            return False
        seq.blocks.extend(self.pool.alloc(need))
        return True

    def _release(self, seq: Sequence, publish: bool) -> None:
        """Give back everything ``seq`` owns; optionally publish its computed full blocks first."""
        if publish and self.radix is not None and seq.blocks:
            n_full = min(seq.num_computed // self.bs, len(seq.blocks))
            if n_full:
                self.radix.insert(seq.all_tokens[:n_full * self.bs], seq.blocks[:n_full], seq.namespace)
        if self.radix is not None and seq.pinned_nodes:
            self.radix.release(seq.pinned_nodes)
        seq.pinned_nodes = []
        if seq.blocks:
            self.pool.free(seq.blocks)
        seq.blocks = []
        if seq.state_slot is not None and self.state_pool is not None:
            self.state_pool.free(seq.state_slot)
        seq.state_slot, seq.has_state = None, False
        seq.drafts = []
        if seq.host_blocks or seq.host_state is not None or seq.disk_blocks:
            self.host_tier.free(seq.host_blocks)
            self.host_tier.free_state(seq.host_state)
            if seq.disk_blocks:
                self.host_tier.disk.free(seq.disk_blocks)
            seq.host_blocks, seq.host_state, seq.disk_blocks = [], None, []

    def _spill_to_disk(self, need_host: int, out: SchedulerOutput, keep: Optional[Sequence] = None) -> bool:
        """Free ``need_host`` host blocks by moving parked sequences to the disk tier, starting with the one whose turn
        to resume is furthest away.  The engine writes the records before any copy that reuses the host blocks."""
        ht = self.host_tier
        disk = getattr(ht, "disk", None)
        if disk is None:
            return ht.num_free >= need_host
        for seq in reversed(self.swapped):
            if ht.num_free >= need_host:
                break
            if seq is keep or not seq.host_blocks or disk.num_free < len(seq.host_blocks):
                continue
            records = disk.alloc(len(seq.host_blocks))
            out.disk_out.append((list(seq.host_blocks), list(records)))
            ht.free(seq.host_blocks)
            seq.host_blocks, seq.disk_blocks = [], records
            self.num_spills += 1
        return ht.num_free >= need_host

    def _try_swap_out(self, victim: Sequence, out: SchedulerOutput) -> bool:
        """Park a decoding sequence's computed KV (and recurrent state) in the host tier.  Only sequences whose
        context is fully computed qualify; the engine copies before anything else touches the released blocks."""
        ht = self.host_tier
        if ht is None or victim not in self.running or victim.num_computed <= 0 or victim in self._resumed_now:
            return False
        n_used = min(self.pool.blocks_for_tokens(victim.num_computed), len(victim.blocks))
        need_state = self.hybrid and victim.state_slot is not None
        if need_state and ht.num_free_states == 0:
            return False
        if ht.num_free < n_used and not self._spill_to_disk(n_used, out):
            return False
        host_blocks = ht.alloc(n_used)
        host_state = ht.alloc_state() if need_state else None
        out.swap_out.append((list(victim.blocks[:n_used]), list(host_blocks), victim.state_slot, host_state))
        self.running.remove(victim)
        keep_computed, had_state = victim.num_computed, victim.has_state
        self._release(victim, publish=True)
        victim.host_blocks, victim.host_state = host_blocks, host_state
        victim.num_computed, victim.has_state = keep_computed, had_state
        victim.status = SeqStatus.SWAPPED
        victim.num_preemptions += 1
        self.num_swaps += 1
        self.swapped.append(victim)
        return True

    def _resume_swapped(self, out: SchedulerOutput) -> None:
        """Bring parked sequences back (oldest first) while blocks for their context plus the admission headroom are
        available; they rejoin the decode set of this very step."""
        while self.swapped:
            seq = self.swapped[0]
            if self.num_unfinished - len(self.waiting) - len(self.swapped) >= self.cfg.max_num_seqs:
                return
            if self.hybrid and self.state_pool is not None and seq.host_state is not None and self.state_pool.num_free == 0:
                return
            need = self._admission_blocks(seq, 0)
            avail = self.pool.num_free + (self.radix.evictable_blocks() if self.radix is not None else 0)
            n_used = len(seq.host_blocks) + len(seq.disk_blocks)
            if need > avail:
                return
            if seq.disk_blocks:
                # back through host blocks: the engine reads the records into them before the host -> device copy
                ht = self.host_tier
                if ht.num_free < n_used and not self._spill_to_disk(n_used, out, keep=seq):
                    return
                seq.host_blocks = ht.alloc(n_used)
                out.disk_in.append((list(seq.disk_blocks), list(seq.host_blocks)))
                seq.disk_blocks = []                  # the engine returns the records to the disk tier after reading
            if not self._reclaim(n_used):
                return
            self.swapped.popleft()
            seq.blocks = self.pool.alloc(n_used)
            slot = None
            if seq.host_state is not None:
                slot = self.state_pool.alloc()
                seq.state_slot = slot
            out.swap_in.append((list(seq.host_blocks), list(seq.blocks), seq.host_state, slot))
            seq.host_blocks, seq.host_state = [], None       # the engine returns them to the tier after the copy
            seq.status = SeqStatus.RUNNING
            self.running.append(seq)
            self._resumed_now.append(seq)

    def _preempt(self, victim: Sequence, out: SchedulerOutput) -> None:
        if self._try_swap_out(victim, out):
            return
        (self.running if victim in self.running else self.prefilling).remove(victim)
        # hybrid sequences cannot resume from KV alone; their published blocks only help at snapshot depths
        self._release(victim, publish=True)
        victim.status = SeqStatus.PREEMPTED
        victim.num_computed = 0
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
        out.preempted.append(victim)

    # ------------------------------------------------------------------ admission
    def _admission_blocks(self, seq: Sequence, cached_tokens: int) -> int:
        remaining_out = max(0, seq.sampling.max_tokens - seq.num_output_tokens)
        headroom = min(remaining_out, self.cfg.admission_watermark_tokens)
        total = self.pool.blocks_for_tokens(seq.num_tokens + headroom)
        return total - cached_tokens // self.bs

    def _outstanding_prefill_blocks(self) -> int:
        """Blocks that already-admitted prefills still have to allocate for their prompts.  Admission counts them as
        taken: a prompt admitted on blocks an earlier, partly allocated prefill needs would leave both stuck."""
        short = 0
        for s in self.prefilling:
            short += max(0, self.pool.blocks_for_tokens(s.num_tokens) - len(s.blocks))
        return short

    def _try_admit(self, seq: Sequence, out: SchedulerOutput) -> bool:
        if self.hybrid and self.state_pool is not None and self.state_pool.num_free == 0:
            return False
        match = None
        cached = 0
        if self.radix is not None and self.cfg.enable_prefix_caching:
            match = self.radix.match(seq.all_tokens, seq.namespace, need_snapshot=self.hybrid)
            cached = match.num_tokens
        need = self._admission_blocks(seq, cached)
        avail = self.pool.num_free + (self.radix.evictable_blocks() if self.radix is not None else 0)
        avail -= self._outstanding_prefill_blocks()
        if need > avail:
            if match is not None and match.nodes:
                self.radix.release(match.nodes)
                self.pool.free(match.blocks)
            return False
        if match is not None:
            seq.blocks = list(match.blocks)
            seq.pinned_nodes = list(match.nodes)
        seq.num_computed = cached
        seq.num_cached_tokens = cached
        if self.hybrid and self.state_pool is not None:
            seq.state_slot = self.state_pool.alloc()
            seq.has_state = False
            if match is not None and match.snapshot_slot is not None:
                out.restored_snapshots.append((match.snapshot_slot, seq.state_slot))
                seq.has_state = True
        seq.status = SeqStatus.PREFILL
        if seq.first_scheduled_time is None:
            seq.first_scheduled_time = time.monotonic()
        self.prefilling.append(seq)
        return True

    # ------------------------------------------------------------------ planning
    def schedule(self, now: Optional[float] = None, expire: bool = True) -> SchedulerOutput:
        """``now`` / ``expire=False`` let a multi-process leader impose its clock and its expiry decisions on the
        follower replicas so that every rank plans the same step."""
        out = SchedulerOutput()
        cfg = self.cfg
        now = time.monotonic() if now is None else now
        if expire:
            self._expire_deadlines(now)
        if self._last_decode_time is None:
            self._last_decode_time = now

        # 0. sequences parked in the host tier come back before anything new is admitted
        self._resumed_now = []
        if self.swapped:
            self._resume_swapped(out)

        # 1. decodes (+ draft rows)
        decode_items: List[ScheduledSeq] = []
        i = 0
        while i < len(self.running) and len(decode_items) < cfg.max_batch_size:
            seq = self.running[i]
            n_rows = 1 + len(seq.drafts)
            ok = self._ensure_blocks(seq, seq.num_computed + n_rows)
            while not ok:
                victim = self._pick_victim(exclude=seq)
                if victim is None:
                    break
                decode_items = [d for d in decode_items if d.seq is not victim]
                if victim in self.running and self.running.index(victim) < i:
                    i -= 1
                self._preempt(victim, out)
                ok = self._ensure_blocks(seq, seq.num_computed + n_rows)
            if ok:
                decode_items.append(ScheduledSeq(seq, seq.num_computed, n_rows, True, n_rows == 1, len(seq.drafts)))
                i += 1
            else:
                self._preempt(seq, out)      # nothing left to evict: this one waits too
        budget = self.policy.prefill_budget(cfg.max_prefill_tokens, len(decode_items), now - self._last_decode_time)

        # 2. continue prefills
        prefill_items: List[ScheduledSeq] = []
        for seq in list(self.prefilling):
            if budget <= 0:
                break
            item = self._plan_prefill_chunk(seq, budget, out, len(decode_items) + len(prefill_items))
            if item is None:
                continue
            prefill_items.append(item)
            budget -= item.num_tokens

        # 3. admit new requests (not while the memory watchdog holds admission: running work drains first)
        if self.waiting and not self.admission_paused:
            order = self.policy.order(list(self.waiting))
            for seq in order:
                if budget <= 0 or self.num_unfinished - len(self.waiting) >= cfg.max_num_seqs:
                    break
                if not self._try_admit(seq, out):
                    if self.policy.head_of_line_blocking:
                        break
                    continue
                self.waiting.remove(seq)
                item = self._plan_prefill_chunk(seq, budget, out, len(decode_items) + len(prefill_items))
                if item is not None:
                    prefill_items.append(item)
                    budget -= item.num_tokens

        # Nothing could be planned although prompts are in flight: every free block is held by partly allocated prefills
        # and no decode ran that could have picked a victim.  The youngest prefill gives its blocks back (computed full
        # blocks go to the prefix cache first) so that the oldest one can finish.
        if not decode_items and not prefill_items and len(self.prefilling) > 1 and budget > 0:
            self._preempt(self.prefilling[-1], out)
            item = self._plan_prefill_chunk(self.prefilling[0], budget, out, 0)
            if item is not None:
                prefill_items.append(item)

        # verify rows (q_len > 1) are not "decodes" for the attention kernels: order pure decodes first
        pure = [d for d in decode_items if d.is_decode]
        verify = [d for d in decode_items if not d.is_decode]
        out.items = pure + verify + prefill_items
        if decode_items:
            self._last_decode_time = now
        return out

    def _pick_victim(self, exclude: Sequence) -> Optional[Sequence]:
        for pool in (self.prefilling, self.running):
            for s in reversed(pool):
                if s is not exclude and s not in self._resumed_now:
                    return s
        return None

    def _plan_prefill_chunk(self, seq: Sequence, budget: int, out: SchedulerOutput, item_index: int) -> Optional[ScheduledSeq]:
        remaining = seq.num_uncomputed
        n = min(remaining, budget)
        if n <= 0:
            return None
        if n < remaining and n >= self.bs:
            n = n // self.bs * self.bs if (seq.num_computed % self.bs == 0) else n   # keep chunk ends block aligned
        if not self._ensure_blocks(seq, seq.num_computed + n):
            # shrink to what fits; if nothing fits leave it for a later step
            fit = (len(seq.blocks) + self.pool.num_free) * self.bs - seq.num_computed
            n = min(n, fit)
            if n <= 0 or not self._ensure_blocks(seq, seq.num_computed + n):
                return None
        last = (seq.num_computed + n) == seq.num_tokens
        if self.hybrid and self.radix is not None and self.cfg.enable_prefix_caching and seq.state_slot is not None:
            self._plan_snapshots(seq, n, out, item_index)
        return ScheduledSeq(seq, seq.num_computed, n, last, False)

    def _plan_snapshots(self, seq: Sequence, n: int, out: SchedulerOutput, item_index: int) -> None:
        """Recurrent-state snapshots at block-aligned prompt depths inside this chunk: every
        ``snapshot_interval`` tokens and at the deepest aligned boundary that still leaves one token."""
        lo, hi = seq.num_computed, seq.num_computed + n
        limit = (seq.num_tokens - 1) // self.bs * self.bs
        points = set(p for p in range((lo // self.snapshot_interval + 1) * self.snapshot_interval, hi + 1, self.snapshot_interval)
                     if p <= limit)
        if lo < limit <= hi:
            points.add(limit)
        toks = seq.all_tokens
        for p in sorted(points):
            nodes = self.radix.insert(toks[:p], seq.blocks[:p // self.bs], seq.namespace)
            if not nodes:
                continue
            slot = self.radix.attach_snapshot(nodes[-1])
            if slot is not None:
                out.snapshot_requests.append((item_index, p - lo, slot))

    def expire(self, now: float) -> List[Sequence]:
        """Expire deadlines now; returns the sequences that timed out (they are also queued as finished)."""
        n0 = len(self.finished_queue)
        self._expire_deadlines(now)
        return self.finished_queue[n0:]

    def _expire_deadlines(self, now: float) -> None:
        for q in (self.waiting, self.prefilling, self.running, self.swapped):
            for s in list(q):
                if s.deadline is not None and now > s.deadline:
                    q.remove(s)
                    self._release(s, publish=False)
                    s.status, s.finish_reason, s.finish_time = SeqStatus.FINISHED, FinishReason.TIMEOUT, now
                    self.finished_queue.append(s)

    # ------------------------------------------------------------------ step results
    def on_chunk_computed(self, item: ScheduledSeq, num_rows_kept: Optional[int] = None) -> None:
        """Advance ``num_computed`` after the forward pass (``num_rows_kept`` < rows for rejected drafts)."""
        seq = item.seq
        seq.num_computed += item.num_tokens if num_rows_kept is None else num_rows_kept
        if self.hybrid:
            seq.has_state = True

    def promote(self, seq: Sequence) -> None:
        """PREFILL -> RUNNING once the whole prompt (or resume context) is computed and a token sampled."""
        if seq in self.prefilling:
            self.prefilling.remove(seq)
            seq.status = SeqStatus.RUNNING
            self.running.append(seq)

    def finish(self, seq: Sequence, reason: FinishReason) -> None:
        for q in (self.prefilling, self.running):
            if seq in q:
                q.remove(seq)
        self._release(seq, publish=self.cfg.enable_prefix_caching)
        seq.status, seq.finish_reason, seq.finish_time = SeqStatus.FINISHED, reason, time.monotonic()

    def trim_blocks(self, seq: Sequence) -> None:
        """Return blocks past the computed length (after rejected speculative rows)."""
        keep = self.pool.blocks_for_tokens(max(seq.num_computed + 1, 1))
        if len(seq.blocks) > keep:
            extra = seq.blocks[keep:]
            del seq.blocks[keep:]
            seq._blocks_cache = None        # the runner's array view of the table is stale now
            self.pool.free(extra)

    def snapshot(self) -> Dict[str, int]:
        return {"waiting": len(self.waiting), "prefilling": len(self.prefilling), "running": len(self.running),
                "kv_free_blocks": self.pool.num_free, "kv_total_blocks": self.pool.num_blocks,
                "preemptions": self.num_preemptions, "swapped": len(self.swapped), "swaps": self.num_swaps,
                "state_slots_free": self.state_pool.num_free if self.state_pool else 0}
