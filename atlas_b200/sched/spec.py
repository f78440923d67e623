"""Speculative decoding control: MTP proposal chain, acceptance bookkeeping and the throughput gate.

Per step, after the target model has run and tokens were sampled:

1. the MTP head consumes ``(target hidden at p, token at p+1)`` for every row the step kept, which
   keeps the head's own KV layer in lock-step with the target's;
2. for sequences that just emitted a token the head's last row gives draft ``d1``; ``d2..dK`` come from
   a chain of single-row head steps fed with the head's own hidden;
3. the next engine step verifies ``[last, d1..dK]`` as K+1 query rows; a draft is accepted while it
   equals the token the target samples at that row (so emitted tokens are exactly the target's).

The gate arbitrates between speculative and plain decoding by measured emitted tokens per second,
re-measuring the losing mode periodically.

Reference parity: ``crates/spark-server/src/scheduler/mtp_step.rs``, ``mtp_gate.rs`` (MeasureDecode /
MeasureVerify arbitration), ``crates/spark-model/src/speculative.rs:327`` (``DraftProposer``),
``layers/mtp_head/propose_chain.rs``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config import EngineConfig
from ..models import ForwardBatch
from .sequence import SchedulerOutput, SeqStatus


class MtpGate:
    """Throughput arbitration between speculative and plain decode."""

    def __init__(self, enabled: bool = True, window: int = 32, remeasure_every: int = 512, probe_steps: int = 16, agree=None):
        """``agree``: maps this rank's ``[seconds, tokens]`` of a finished probe to the values every rank uses (e.g. a
        MAX all-reduce).  Ranks that run the same engine loop side by side time their steps a little differently; without
        an agreed measurement they would pick different modes and issue different collectives."""
        self.enabled = enabled
        self.agree = agree
        self.window, self.remeasure_every, self.probe_steps = window, remeasure_every, probe_steps
        self.mode = "spec"                       # spec | plain
        self.tps = {"spec": 0.0, "plain": 0.0}
        self._acc = {"spec": [0.0, 0], "plain": [0.0, 0]}   # [seconds, tokens]
        self._steps_in_mode = 0
        self._probing: Optional[str] = "spec" if enabled else None
        self._since_measure = 0

    def use_spec(self) -> bool:
        if not self.enabled:
            return True
        return (self._probing or self.mode) == "spec"

    def record(self, was_spec: bool, seconds: float, tokens: int) -> None:
        if not self.enabled or tokens <= 0:
            return
        key = "spec" if was_spec else "plain"
        acc = self._acc[key]
        acc[0] += seconds
        acc[1] += tokens
        self._steps_in_mode += 1
        self._since_measure += 1
        if self._probing is not None and self._steps_in_mode >= self.probe_steps:
            sec, tok = self._acc[self._probing]
            if self.agree is not None:
                sec, tok = self.agree([sec, float(tok)])
            if sec > 0:
                self.tps[self._probing] = tok / sec
            self._acc[self._probing] = [0.0, 0]
            self._steps_in_mode = 0
            if self._probing == "spec" and self.tps["plain"] == 0.0:
                self._probing = "plain"
            else:
                self._probing = None
                self.mode = "spec" if self.tps["spec"] >= self.tps["plain"] else "plain"
                self._since_measure = 0
        elif self._probing is None and self._since_measure >= self.remeasure_every:
            self._probing = "plain" if self.mode == "spec" else "spec"
            self._steps_in_mode = 0
            self._acc[self._probing] = [0.0, 0]


def rank_agreement(engine):
    """The gate's ``agree`` hook for ranks that run the engine loop symmetrically (tensor / expert parallel without a
    leader process): a MAX all-reduce of the probe measurement over the default process group.  None for one process or
    when a leader imposes its decisions anyway."""
    p = getattr(getattr(engine, "model", None), "pctx", None)
    if p is None or getattr(engine, "control", None) is not None or max(p.tp_size, p.ep_size) <= 1:
        return None
    try:
        import torch.distributed as dist
        if not dist.is_initialized():
            return None
    except Exception:
        return None
    dev = engine.model.device

    def agree(vals):
        t = torch.tensor(vals, dtype=torch.float64, device=dev if dev.type == "cuda" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()
    return agree


class SpecController:
    def __init__(self, engine, cfg: EngineConfig):
        self.engine = engine
        self.cfg = cfg
        self.k = cfg.num_drafts
        self.gate = MtpGate(enabled=cfg.mtp_gate, agree=rank_agreement(engine))
        self.dcut_pruned = 0                     # draft rows dropped by the verify-depth planner

    def active(self) -> bool:
        return True

    # ------------------------------------------------------------------ after each target step
    @torch.inference_mode()
    def after_step(self, out: SchedulerOutput, batch: ForwardBatch, hidden: torch.Tensor,
                   sampled: Dict[int, List[int]], kept_rows: List[int]) -> None:
        eng = self.engine
        model, mtp, runner = eng.model, eng.model.mtp, eng.runner
        bs = eng.cfg.block_size
        rows: List[int] = []
        toks: List[List[int]] = []
        ctxs: List[int] = []
        tables: List[List[int]] = []
        owners: List[int] = []
        propose: List[bool] = []
        r0 = 0
        for idx, it in enumerate(out.items):
            seq = it.seq
            m = kept_rows[idx]
            n_in = it.num_tokens
            if seq.finished or m <= 0:
                r0 += n_in
                continue
            all_toks = seq.all_tokens
            nxt = all_toks[it.start + 1:it.start + m + 1]        # token at p+1 for each kept row p
            if len(nxt) < m:
                r0 += n_in
                continue
            rows.extend(range(r0, r0 + m))
            toks.append(nxt)
            ctxs.append(it.start)
            tables.append(seq.blocks)
            owners.append(idx)
            propose.append(bool(it.sample) and seq.status == SeqStatus.RUNNING and not seq.disable_spec)
            r0 += n_in
        if not rows:
            return
        fb = ForwardBatch.build(toks, ctxs, tables, bs, device=model.device)
        fb.num_decodes = 0          # positions are arbitrary chunks; use the general attention path
        ridx = torch.tensor(rows, dtype=torch.long, device=hidden.device)
        h_prev = hidden[ridx]
        emb = model.embed_tokens(fb.input_ids)
        mh = mtp.forward(fb, emb, h_prev, eng.cache, model.rope_cache)
        last_rows = (fb.query_start_loc[1:] - 1).long()
        want = [i for i, p in enumerate(propose) if p]
        if not want or not self.gate.use_spec():
            return
        sel = last_rows[torch.tensor(want, device=last_rows.device)]
        cur_h = mh[sel]
        drafts: List[List[int]] = [[] for _ in want]
        seqs = [out.items[owners[i]].seq for i in want]
        dcut_on = self.cfg.dcut_ratio > 0
        conf: List[List[float]] = [[] for _ in want]            # ln of the drafter's top-1 probability per draft

        def top1(h):
            tok, lp = model.draft_top1(h, want_logprob=dcut_on)      # the reduced draft head when the model has one
            return tok.tolist(), (lp.tolist() if lp is not None else None)
        d, lp0 = top1(cur_h)
        for j, t in enumerate(d):
            drafts[j].append(int(t))
            if lp0 is not None:
                conf[j].append(float(lp0[j]))
        alive = list(range(len(want)))
        for step in range(1, self.k):
            # chain: position p+step, inputs (head hidden, previous draft)
            ok = [j for j in alive if eng.scheduler._ensure_blocks(seqs[j], seqs[j].num_computed + step)]
            if not ok:
                break
            alive = ok
            t_in = [[drafts[j][-1]] for j in alive]
            c_in = [seqs[j].num_computed + step - 1 for j in alive]
            fbc = ForwardBatch.build(t_in, c_in, [seqs[j].blocks for j in alive], bs, device=model.device)
            fbc.num_decodes = 0
            hsel = cur_h[torch.tensor(alive, device=cur_h.device)] if len(alive) != cur_h.shape[0] else cur_h
            mh2 = mtp.forward(fbc, model.embed_tokens(fbc.input_ids), hsel, eng.cache, model.rope_cache)
            d, lpn = top1(mh2)
            nh = cur_h.clone()
            for jj, j in enumerate(alive):
                drafts[j].append(int(d[jj]))
                if lpn is not None:
                    conf[j].append(float(lpn[jj]))
                nh[j] = mh2[jj]
            cur_h = nh
        keep = [len(x) for x in drafts]
        if dcut_on:
            from . import dcut
            keep = dcut.plan(conf, self.cfg.dcut_ratio)        # verify depth per sequence from the drafter's confidence
            self.dcut_pruned += sum(len(x) for x in drafts) - sum(keep)
        for j, s in enumerate(seqs):
            room = s.sampling.max_tokens - s.num_output_tokens - 1
            s.drafts = drafts[j][:max(0, min(self.k, room, keep[j]))]


class NgramSpecController:
    """Draft tokens by prompt lookup: find the longest recent n-gram (``ngram_max`` .. ``ngram_min`` tokens ending at
    the sequence's last token) that occurred earlier in the prompt or the output and propose the tokens that followed it.
    No draft model is involved, so it works for every architecture; verification, acceptance (match against the target's
    own samples), write-on-accept state handling and the throughput gate are the ones the MTP path uses.

    The index (n-gram -> position after its latest earlier occurrence) is kept per sequence and extended by the tokens
    appended since the last step.  Reference parity: ``crates/spark-server/src/ngram.rs`` (prompt-lookup proposer),
    ``scheduler/spec_step.rs`` (n-gram / self-speculative step), ``scheduler/copy_draft/``.
    """

    def __init__(self, engine, cfg: EngineConfig):
        self.engine, self.cfg = engine, cfg
        self.k = max(1, cfg.num_drafts)
        self.n_max, self.n_min = max(1, cfg.ngram_max), max(1, min(cfg.ngram_min, cfg.ngram_max))
        self.gate = MtpGate(enabled=cfg.mtp_gate, agree=rank_agreement(engine))
        self.proposed_steps = 0

    def active(self) -> bool:
        return True

    def _index(self, seq):
        st = getattr(seq, "_ngram_state", None)
        if st is None:
            st = seq._ngram_state = {"upto": 0, "maps": {n: {} for n in range(self.n_min, self.n_max + 1)}}
        return st

    def propose(self, seq) -> List[int]:
        total = seq.num_tokens
        st = self._index(seq)
        tok = seq.token_at
        # index every n-gram that ENDS before the last token, so a lookup never matches itself
        for end in range(max(st["upto"], self.n_min), total):          # gram = tokens[end-n:end]; what follows starts at `end`
            for n, mp in st["maps"].items():
                if end - n >= 0:
                    mp[tuple(tok(i) for i in range(end - n, end))] = end
        st["upto"] = max(st["upto"], total)
        for n in range(self.n_max, self.n_min - 1, -1):
            if total < n:
                continue
            pos = st["maps"][n].get(tuple(tok(i) for i in range(total - n, total)))
            if pos is not None and pos < total:
                return [tok(i) for i in range(pos, min(pos + self.k, total))]
        return []

    def after_step(self, out: SchedulerOutput, batch: ForwardBatch, hidden, sampled, kept_rows) -> None:
        if not self.gate.use_spec():
            return
        any_draft = False
        for it in out.items:
            seq = it.seq
            if seq.finished or seq.status != SeqStatus.RUNNING or seq.disable_spec or not it.sample:
                continue
            room = seq.sampling.max_tokens - seq.num_output_tokens - 1
            drafts = self.propose(seq)[:max(0, min(self.k, room))]
            seq.drafts = drafts
            any_draft |= bool(drafts)
        self.proposed_steps += 1 if any_draft else 0


class DFlashSpecController:
    """Drafts from the block-diffusion draft model (``models/dflash.py``): after every target step the states of the
    captured target layers at the kept rows become context keys / values of the drafter, then ONE drafter forward per
    step proposes ``num_drafts`` tokens for every decoding sequence.  Verification, acceptance and the throughput gate
    are shared with the other proposers.  Reference parity: ``crates/spark-model/src/layers/dflash_head/propose.rs``,
    ``crates/spark-server/src/scheduler/spec_step.rs``."""

    def __init__(self, engine, cfg: EngineConfig):
        self.engine, self.cfg = engine, cfg
        self.k = max(1, cfg.num_drafts)
        self.gate = MtpGate(enabled=cfg.mtp_gate, agree=rank_agreement(engine))
        self.drafter = engine.model.dflash
        self.proposed_steps = 0

    def active(self) -> bool:
        return True

    @torch.inference_mode()
    def after_step(self, out: SchedulerOutput, batch: ForwardBatch, hidden, sampled, kept_rows) -> None:
        eng, model, d = self.engine, self.engine.model, self.drafter
        bs = eng.cfg.block_size
        aux = model.aux_hidden
        if len(aux) != len(d.dcfg.target_layer_ids):
            return
        rows, pos, slots = [], [], []
        want = []
        r0 = 0
        for idx, it in enumerate(out.items):
            seq, m, n_in = it.seq, kept_rows[idx], it.num_tokens
            if not seq.finished and m > 0:
                for j in range(m):
                    p = it.start + j
                    rows.append(r0 + j)
                    pos.append(p)
                    slots.append(seq.blocks[p // bs] * bs + p % bs)
                if (it.sample and seq.status == SeqStatus.RUNNING and not seq.disable_spec
                        and seq.num_tokens == it.start + m + 1):
                    want.append((seq, it.start + m))
            r0 += n_in
        if rows:
            ridx = torch.tensor(rows, dtype=torch.long, device=model.device)
            feats = d.context_features([a[ridx] for a in aux])
            d.add_context(feats, torch.tensor(pos, dtype=torch.int32, device=model.device),
                          torch.tensor(slots, dtype=torch.int32, device=model.device))
        if not want or not self.gate.use_spec():
            return
        ready = []
        for seq, ctx in want:
            room = seq.sampling.max_tokens - seq.num_output_tokens - 1
            k = max(0, min(self.k, room))
            if k > 0 and eng.scheduler._ensure_blocks(seq, ctx + self.k + 1):
                ready.append((seq, ctx, k))
        if not ready:
            return
        drafts = d.propose([s.token_at(c) for s, c, _ in ready], [c for _, c, _ in ready], [s.blocks for s, _, _ in ready], self.k)
        for (seq, _, k), dr in zip(ready, drafts):
            seq.drafts = dr[:k]
        self.proposed_steps += 1


def skip_layer_ids(num_layers: int, keep: float) -> List[int]:
    """The layers a layer-skipping draft pass runs: the first and the last layer and an even spread in between."""
    n_keep = max(2, min(num_layers, int(round(num_layers * keep)))) if num_layers > 1 else 1
    if n_keep >= num_layers:
        return list(range(num_layers))
    ids = sorted({round(i * (num_layers - 1) / (n_keep - 1)) for i in range(n_keep)})
    return [int(i) for i in ids]


class SelfSpecController:
    """Self-speculative decoding: the drafts come from the target model itself, run with most layers skipped.  After
    every target step the sequences that just sampled a token take ``num_drafts`` chained draft steps through the kept
    layers (one batched forward per step; the kept layers write their KV entries at the draft positions, which the
    verify step recomputes and overwrites together with everybody else's), and the next target step verifies the
    chain.  No extra weights, so it applies to every attention-only checkpoint; models with recurrent layers are left
    out (a draft pass would advance their state).  Verification, acceptance and the throughput gate are shared with the
    other proposers.  Reference parity: ``crates/spark-model/src/model/trait_impl/speculative.rs`` (layer-skipping
    draft, ``generate_self_speculative_inner``), ``crates/spark-server/src/scheduler/spec_step.rs::step_self_spec``."""

    def __init__(self, engine, cfg: EngineConfig):
        self.engine, self.cfg = engine, cfg
        self.k = max(1, cfg.num_drafts)
        self.gate = MtpGate(enabled=cfg.mtp_gate, agree=rank_agreement(engine))
        self.layer_ids = skip_layer_ids(len(engine.model.layers), cfg.self_spec_keep)
        self.proposed_steps = 0

    @staticmethod
    def supported(model) -> bool:
        return all(getattr(l, "kind", None) == "attention" for l in model.layers) and not getattr(model, "capture_layers", ())

    def active(self) -> bool:
        return True

    @torch.inference_mode()
    def after_step(self, out: SchedulerOutput, batch: ForwardBatch, hidden, sampled, kept_rows) -> None:
        if not self.gate.use_spec():
            return
        eng, model = self.engine, self.engine.model
        bs = eng.cfg.block_size
        want = []
        for idx, it in enumerate(out.items):
            seq, m = it.seq, kept_rows[idx]
            if (seq.finished or m <= 0 or not it.sample or seq.status != SeqStatus.RUNNING or seq.disable_spec
                    or seq.num_tokens != it.start + m + 1):
                continue
            room = seq.sampling.max_tokens - seq.num_output_tokens - 1
            k = max(0, min(self.k, room))
            if k > 0 and eng.scheduler._ensure_blocks(seq, it.start + m + self.k + 1):
                want.append((seq, it.start + m, k))
        if not want:
            return
        seqs = [w[0] for w in want]
        drafts: List[List[int]] = [[] for _ in want]
        cur = [s.token_at(c) for s, c, _ in want]             # the token the target just sampled, at position c
        for step in range(self.k):
            fb = ForwardBatch.build([[t] for t in cur], [c + step for _, c, _ in want], [s.blocks for s in seqs], bs,
                                    device=model.device)
            h = model.forward(fb, eng.cache, layer_ids=self.layer_ids)
            cur = [int(t) for t in ops.argmax(model.compute_logits(h)).tolist()]
            for j, t in enumerate(cur):
                drafts[j].append(t)
        for (seq, _, k), dr in zip(want, drafts):
            seq.drafts = dr[:k]
        self.proposed_steps += 1
