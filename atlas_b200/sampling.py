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

    @torch.inference_mode()
    def __call__(self, logits: torch.Tensor, seqs: Sequence["object"]) -> SamplerOutput:
        """``logits [B,V]`` (one row per sequence, same order)."""
        B = logits.shape[0]
        assert B == len(seqs)
        if self.fast_greedy(seqs):
            return SamplerOutput(ops.argmax(logits).tolist())
        lf = logits.float().clone()
        dev = lf.device
        for i, s in enumerate(seqs):
            p: SamplingParams = s.sampling
            if p.logit_bias:
                idx = torch.tensor(list(p.logit_bias.keys()), device=dev, dtype=torch.long)
                lf[i, idx] += torch.tensor(list(p.logit_bias.values()), device=dev, dtype=torch.float32)
            if p.min_tokens > 0 and s.num_output_tokens < p.min_tokens:
                stop_ids = list(self.eos_ids) + list(p.stop_token_ids)
                if stop_ids:
                    lf[i, torch.tensor(stop_ids, device=dev, dtype=torch.long)] = float("-inf")
            if s.grammar is not None:
                mask = s.grammar.token_mask(self.vocab)
                if mask is not None:
                    lf[i] = lf[i].masked_fill(~mask.to(dev), float("-inf"))
            for proc in s.logits_processors:
                lf[i] = proc(lf[i], s)
            if p.needs_penalties:
                lf[i] = self._penalise_row(lf[i], s)
            if p.top_n_sigma > 0:
                lf[i] = top_n_sigma_mask(lf[i:i + 1], p.top_n_sigma)[0]
        temp = torch.tensor([s.sampling.temperature for s in seqs], dtype=torch.float32, device=dev)
        if bool((temp <= 0).all()):
            toks = ops.argmax(lf)
        else:
            top_k = torch.tensor([s.sampling.top_k for s in seqs], dtype=torch.int32, device=dev)
            top_p = torch.tensor([s.sampling.top_p for s in seqs], dtype=torch.float32, device=dev)
            min_p = torch.tensor([s.sampling.min_p for s in seqs], dtype=torch.float32, device=dev)
            u = torch.tensor([s.rng.uniform(s.num_output_tokens) for s in seqs], dtype=torch.float32, device=dev)
            toks = ops.sample(lf, temp, top_k, top_p, min_p, u)
        toks_l = toks.tolist()
        lps = None
        if any(s.sampling.logprobs for s in seqs):
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
        return SamplerOutput(toks_l, lps)

    def _penalise_row(self, row: torch.Tensor, s) -> torch.Tensor:
        p: SamplingParams = s.sampling
        dev = row.device
        out_toks = s.output_tokens
        hist = s.prompt_tokens + out_toks
        if p.repetition_window > 0:
            hist = hist[-p.repetition_window:]
        if p.repetition_penalty != 1.0 and hist:
            idx = torch.tensor(sorted(set(hist)), device=dev, dtype=torch.long)
            vals = row[idx]
            row[idx] = torch.where(vals > 0, vals / p.repetition_penalty, vals * p.repetition_penalty)
        if (p.presence_penalty or p.frequency_penalty) and out_toks:
            counts: Dict[int, int] = {}
            for t in out_toks:
                counts[t] = counts.get(t, 0) + 1
            idx = torch.tensor(list(counts.keys()), device=dev, dtype=torch.long)
            c = torch.tensor(list(counts.values()), device=dev, dtype=torch.float32)
            row[idx] -= p.frequency_penalty * c + p.presence_penalty
        if p.dry_multiplier > 0:
            pen = dry_penalty(s.prompt_tokens + out_toks, p, self.vocab)
            if pen:
                idx = torch.tensor(list(pen.keys()), device=dev, dtype=torch.long)
                row[idx] -= torch.tensor(list(pen.values()), device=dev, dtype=torch.float32)
        return row
