"""D-Cut: adaptive verification-depth pruning for speculative decoding.

The drafter proposes up to ``k`` tokens per sequence and every proposed token costs one row of the verify forward.
A draft at depth ``j`` only matters if every draft before it is accepted, so its survival score is the prefix product
of the drafter's top-1 probabilities, in log space the prefix sum ``s[i][j] = sum_{t<=j} ln c[i][t]``.  All prunable
positions of the whole batch are ranked by that score and the best ``ratio`` fraction is kept (the ratio snaps to the
buckets 0.25 / 0.5 / 0.75 / 1.0), within a total row budget.  Because log-probabilities are <= 0 the score never
increases with depth, so what is kept is a contiguous prefix per sequence: the result is just a draft count per sequence.
Every sequence keeps at least one draft, and batches wider than ``max_seqs`` are left unpruned.

The cost-model variant picks the budget that maximises expected accepted tokens per unit of verify cost, with the
cost of a verify step modelled as ``base + per_row * rows`` and acceptance estimated from the (calibrated) survival
scores.

Reference parity: ``crates/spark-server/src/scheduler/mtp_dcut.rs`` (``plan``, buckets, row budget, width cap) and
``mtp_dcut_cost.rs`` / ``mtp_accept_estimator.rs``.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

BUCKETS = (0.25, 0.5, 0.75, 1.0)
VERIFY_ROW_BUDGET = 160


def snap_ratio(r: float) -> float:
    return min(BUCKETS, key=lambda b: abs(b - r))


def plan(log_probs: Sequence[Sequence[float]], ratio: float = 0.5, row_budget: int = VERIFY_ROW_BUDGET, max_seqs: int = 8) -> List[int]:
    """``log_probs[i][j]`` = ln of the drafter's top-1 probability of sequence i's draft j.  Returns the number of
    drafts to verify per sequence (each >= 1 when the sequence has drafts)."""
    n = len(log_probs)
    full = [len(lp) for lp in log_probs]
    if n == 0 or n > max_seqs:
        return _fit_budget(full, log_probs, row_budget)
    ratio = snap_ratio(ratio)
    scored = []
    for i, lp in enumerate(log_probs):
        s = 0.0
        for j, v in enumerate(lp):
            s += min(0.0, float(v))
            if j >= 1:                                   # depth 0 is always kept
                scored.append((s, i, j))
    keep_extra = int(math.floor(ratio * len(scored) + 1e-9))
    scored.sort(key=lambda t: (-t[0], t[1], t[2]))
    counts = [min(1, f) for f in full]
    for s, i, j in scored[:keep_extra]:
        counts[i] = max(counts[i], j + 1)
    # a kept position implies all shallower ones of its sequence (scores are non-increasing in depth); make that explicit
    return _fit_budget(counts, log_probs, row_budget)


def _fit_budget(counts: List[int], log_probs, row_budget: int) -> List[int]:
    """Rows = one per kept draft plus the sequence's own row; trim the weakest deepest drafts until they fit."""
    counts = list(counts)

    def rows():
        return sum(c + 1 for c in counts if c > 0)
    while rows() > row_budget:
        worst, wi = None, -1
        for i, c in enumerate(counts):
            if c > 1:
                s = sum(min(0.0, float(v)) for v in log_probs[i][:c])
                if worst is None or s < worst:
                    worst, wi = s, i
        if wi < 0:
            break
        counts[wi] -= 1
    return counts


class AcceptEstimator:
    """Online calibration of survival scores: acceptance frequency per score bucket (exponentially averaged), so that
    ``p_accept(score)`` tracks what the verifier actually accepts rather than what the drafter believes."""

    def __init__(self, buckets: int = 16, lo: float = -8.0, decay: float = 0.98):
        self.n, self.lo, self.decay = buckets, lo, decay
        self.hit = [0.0] * buckets
        self.tot = [0.0] * buckets

    def _b(self, score: float) -> int:
        x = min(0.0, max(self.lo, score))
        return min(self.n - 1, int((x - self.lo) / (-self.lo) * self.n))

    def record(self, score: float, accepted: bool) -> None:
        b = self._b(score)
        self.hit[b] = self.hit[b] * self.decay + (1.0 if accepted else 0.0)
        self.tot[b] = self.tot[b] * self.decay + 1.0

    def p_accept(self, score: float) -> float:
        b = self._b(score)
        if self.tot[b] < 4.0:
            return math.exp(min(0.0, score))              # uncalibrated: trust the drafter
        return self.hit[b] / self.tot[b]


def plan_cost_optimal(log_probs: Sequence[Sequence[float]], est: Optional[AcceptEstimator], base_cost: float, row_cost: float,
                      row_budget: int = VERIFY_ROW_BUDGET, max_seqs: int = 8) -> List[int]:
    """Greedy marginal analysis: add the position with the best survival probability while its expected accepted token
    is worth more than the row it costs at the current tokens-per-cost rate."""
    n = len(log_probs)
    counts = [min(1, len(lp)) for lp in log_probs]
    if n == 0 or n > max_seqs:
        return _fit_budget([len(lp) for lp in log_probs], log_probs, row_budget)
    cand = []
    for i, lp in enumerate(log_probs):
        s = 0.0
        for j, v in enumerate(lp):
            s += min(0.0, float(v))
            p = est.p_accept(s) if est is not None else math.exp(s)
            if j == 0:
                continue
            cand.append((p, i, j))
    cand.sort(key=lambda t: (-t[0], t[1], t[2]))

    def p_of(i, j):
        s = sum(min(0.0, float(v)) for v in log_probs[i][:j + 1])
        return est.p_accept(s) if est is not None else math.exp(s)
    tokens = float(n) + sum(p_of(i, 0) for i in range(n) if counts[i])       # the bonus token + depth-0 drafts
    rows = sum(c + 1 for c in counts if c > 0)
    for p, i, j in cand:
        if j != counts[i]:                                # only the next depth of a sequence can be added
            continue
        if rows + 1 > row_budget:
            break
        rate = tokens / (base_cost + row_cost * rows)
        if p < rate * row_cost:                           # the extra row costs more time than its expected token is worth
            break
        counts[i] += 1
        rows += 1
        tokens += p
    return counts
