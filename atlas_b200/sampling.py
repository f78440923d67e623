"""Sampling parameters, the pre-sample logits pipeline and the batched sampler.

The pipeline order is: logit bias -> min-tokens EOS suppression -> grammar / allowed-token masks ->
repetition / presence / frequency (+DRY) penalties -> top-n-sigma -> temperature / top-k / top-p /
min-p sampling (device kernel).  A step where every row is greedy with no penalties or masks takes
the argmax fast path and never materialises probabilities.

Randomness is per request: each request owns a counter-based stream seeded from its ``seed`` so the
token it draws at output position ``i`` does not depend on which other requests share the batch
(order-independence gate).

Reference parity: ``crates/spark-runtime/src/sampler.rs:51-584`` (``SamplingParams``, penalties, DRY
``:324``), ``crates/spark-server/src/scheduler/logit_processors/`` and ``scheduler/fast_greedy.rs``.
"""
from __future__ import annotations

import hashlib
import math
import struct
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from . import ops
from .ops import reference as ref


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    top_n_sigma: float = 0.0
    repetition_penalty: float = 1.0
    repetition_window: int = 0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_breakers: List[int] = field(default_factory=list)
    logit_bias: Dict[int, float] = field(default_factory=dict)
    max_tokens: int = 256
    min_tokens: int = 0
    stop_token_ids: List[int] = field(default_factory=list)
    stop: List[str] = field(default_factory=list)
    ignore_eos: bool = False
    seed: Optional[int] = None
    logprobs: bool = False
    top_logprobs: int = 0
    prompt_logprobs: bool = False
    n: int = 1

    def to_dict(self) -> dict:
        from dataclasses import asdict
        return asdict(self)

    @staticmethod
    def from_dict(d: dict) -> "SamplingParams":
        d = dict(d)
        d["logit_bias"] = {int(k): float(v) for k, v in (d.get("logit_bias") or {}).items()}
        return SamplingParams(**d)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def needs_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or self.dry_multiplier > 0.0)

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not (0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if not (0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be in [0, 1]")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")


class RequestRng:
    """Counter-based uniform stream: ``u_i = H(seed, i)`` — position-addressed, batch-independent."""

    def __init__(self, seed: Optional[int], request_key: str = ""):
        base = seed if seed is not None else int.from_bytes(hashlib.blake2b(request_key.encode(), digest_size=8).digest(), "little")
        self._key = struct.pack("<Q", base & (2 ** 64 - 1))

    def uniform(self, position: int, lane: int = 0) -> float:
        d = hashlib.blake2b(struct.pack("<QI", position, lane), key=self._key, digest_size=8).digest()
        return (int.from_bytes(d, "little") >> 11) / float(1 << 53)


# ----------------------------------------------------------------------------- logits processors
LogitsProcessor = Callable[[torch.Tensor, "object"], torch.Tensor]   # (row logits fp32 [V], sequence) -> logits


def dry_penalty(tokens: Sequence[int], p: SamplingParams, vocab: int) -> Dict[int, float]:
    """DRY ("don't repeat yourself") penalty: for every earlier occurrence of the current suffix, penalise
    the token that followed it by ``multiplier * base ** (match_len - allowed_length)``."""
    out: Dict[int, float] = {}
    n = len(tokens)
    if p.dry_multiplier <= 0 or n < 2:
        return out
    breakers = set(p.dry_breakers)
    last = tokens[-1]
    if last in breakers:
        return out
    for i in range(n - 2, -1, -1):
        if tokens[i] != last:
            continue
        m = 1
        while i - m >= 0 and m < 64 and tokens[i - m] == tokens[n - 1 - m] and tokens[i - m] not in breakers:
            m += 1
        if m >= p.dry_allowed_length:
            nxt = tokens[i + 1]
            pen = p.dry_multiplier * (p.dry_base ** (m - p.dry_allowed_length))
            out[nxt] = max(out.get(nxt, 0.0), pen)
    return out


def top_n_sigma_mask(logits: torch.Tensor, n_sigma: float) -> torch.Tensor:
    """Keep tokens with ``logit >= max - n * std`` (per row)."""
    mx = logits.max(-1, keepdim=True).values
    sd = logits.std(-1, keepdim=True)
    return logits.masked_fill(logits < mx - n_sigma * sd, float("-inf"))


@dataclass
class SamplerOutput:
    tokens: List[int]
    logprobs: Optional[List[Optional[dict]]] = None


class Sampler:
    """Batched sampler over the rows selected for this step."""

    def __init__(self, vocab_size: int, eos_ids: Sequence[int] = ()):
        self.vocab = vocab_size
        self.eos_ids = list(eos_ids)

    def _row_needs_slow_path(self, seq) -> bool:
        p: SamplingParams = seq.sampling
        return (not p.greedy or p.needs_penalties or bool(p.logit_bias) or p.top_n_sigma > 0
                or (p.min_tokens > 0 and seq.num_output_tokens < p.min_tokens)
                or seq.grammar is not None or bool(seq.logits_processors) or p.logprobs
                or getattr(seq, "needs_full_logits", False))

    def fast_greedy(self, seqs: Sequence["object"]) -> bool:
        """True when every row is plain greedy: the step only needs the argmax of each logits row."""
        return not any(self._row_needs_slow_path(s) for s in seqs)

    # ------------------------------------------------------------------ sparse edits (bias, min-tokens, penalties)
    def _row_edits(self, i: int, s, stage_bias: bool, stage_pen: bool, out: Dict[tuple, list]) -> None:
        """Collect this row's (token -> [add, rep, sub, flags]) edits.  ``stage_bias``: logit bias and the min-tokens
        ban; ``stage_pen``: repetition / presence / frequency / DRY penalties."""
        p: SamplingParams = s.sampling

        def slot(tok: int) -> list:
            e = out.get((i, tok))
            if e is None:
                e = out[(i, tok)] = [0.0, 1.0, 0.0, 0]
            return e
        if stage_bias:
            for tok, v in p.logit_bias.items():
                if 0 <= tok < self.vocab:
                    slot(tok)[0] += float(v)
            if p.min_tokens > 0 and s.num_output_tokens < p.min_tokens:
                for tok in list(self.eos_ids) + list(p.stop_token_ids):
                    if 0 <= tok < self.vocab:
                        slot(tok)[3] |= 1
        if stage_pen and p.needs_penalties:
            out_toks = s.output_tokens
            hist = s.prompt_tokens + out_toks
            if p.repetition_window > 0:
                hist = hist[-p.repetition_window:]
            if p.repetition_penalty != 1.0:
                for tok in set(hist):
                    slot(tok)[1] = float(p.repetition_penalty)
            if (p.presence_penalty or p.frequency_penalty) and out_toks:
                counts: Dict[int, int] = {}
                for t in out_toks:
                    counts[t] = counts.get(t, 0) + 1
                for tok, c in counts.items():
                    slot(tok)[2] += p.frequency_penalty * c + p.presence_penalty
            if p.dry_multiplier > 0:
                for tok, pen in dry_penalty(s.prompt_tokens + out_toks, p, self.vocab).items():
                    slot(tok)[2] += pen

    def _apply_edits(self, lf: torch.Tensor, edits: Dict[tuple, list]) -> None:
        """One upload and one kernel for the whole step's edit list."""
        if not edits:
            return
        import numpy as np
        n = len(edits)
        rec = np.empty((n, 6), dtype=np.int32)
        keys = np.fromiter((k for rt in edits.keys() for k in rt), dtype=np.int64, count=2 * n).reshape(n, 2)
        vals = np.asarray(list(edits.values()), dtype=np.float64)
        rec[:, 0:2] = keys
        rec[:, 2:5] = vals[:, 0:3].astype(np.float32).view(np.int32)
        rec[:, 5] = vals[:, 3].astype(np.int32)
        t = torch.from_numpy(rec)
        if lf.is_cuda:
            t = t.pin_memory().to(lf.device, non_blocking=True)
        ops.logit_edits(lf, t)

    @torch.inference_mode()
    def __call__(self, logits: torch.Tensor, seqs: Sequence["object"]) -> SamplerOutput:
        """``logits [B,V]`` (one row per sequence, same order)."""
        toks, lps = self.sample_tensor(logits, seqs)
        return SamplerOutput(toks.tolist(), lps)

    @torch.inference_mode()
    def sample_tensor(self, logits: torch.Tensor, seqs: Sequence["object"]):
        """Like calling the sampler, but the tokens stay on the device (``int64 [B]``); returns ``(tokens, logprobs)``."""
        B = logits.shape[0]
        assert B == len(seqs)
        if self.fast_greedy(seqs):
            return ops.argmax(logits), None
        lf = logits.float().clone()
        dev = lf.device
        # Bias, the min-tokens ban and the penalties are sparse: the whole step's edits go to the device as one list and
        # one kernel applies them.  A mask (-inf) commutes with every one of these edits, so the grammar masks can run
        # after them; only rows with caller-supplied processors keep the two-stage order (bias -> processors -> penalties).
        staged = [i for i, s in enumerate(seqs) if s.logits_processors]
        edits: Dict[tuple, list] = {}
        for i, s in enumerate(seqs):
            self._row_edits(i, s, True, i not in staged, edits)
        self._apply_edits(lf, edits)
        for i, s in enumerate(seqs):
            if s.grammar is not None:
                mask = s.grammar.token_mask(self.vocab)
                if mask is not None:
                    lf[i] = lf[i].masked_fill(~mask.to(dev), float("-inf"))
            for proc in s.logits_processors:
                lf[i] = proc(lf[i], s)
        if staged:
            late: Dict[tuple, list] = {}
            for i in staged:
                self._row_edits(i, seqs[i], False, True, late)
            self._apply_edits(lf, late)
        for i, s in enumerate(seqs):
            if s.sampling.top_n_sigma > 0:
                lf[i] = top_n_sigma_mask(lf[i:i + 1], s.sampling.top_n_sigma)[0]
        if all(s.sampling.temperature <= 0 for s in seqs):
            toks = ops.argmax(lf)
        else:
            # the five per-row sampling parameters travel as one packed upload
            par = torch.tensor([[s.sampling.temperature, float(s.sampling.top_k), s.sampling.top_p, s.sampling.min_p,
                                 s.rng.uniform(s.num_output_tokens)] for s in seqs], dtype=torch.float32)
            if lf.is_cuda:
                par = par.pin_memory().to(dev, non_blocking=True)
            par = par.t().contiguous()
            toks = ops.sample(lf, par[0], par[1].to(torch.int32), par[2], par[3], par[4])
        lps = None
        if any(s.sampling.logprobs for s in seqs):
            toks_l = toks.tolist()
            lps = []
            logp = torch.log_softmax(lf, -1)
            for i, s in enumerate(seqs):
                if not s.sampling.logprobs:
                    lps.append(None)
                    continue
                k = max(0, s.sampling.top_logprobs)
                entry = {"token": toks_l[i], "logprob": float(logp[i, toks_l[i]])}
                if k:
                    tv, ti = torch.topk(logp[i], k)
                    entry["top"] = list(zip(ti.tolist(), tv.tolist()))
                lps.append(entry)
        return toks, lps
