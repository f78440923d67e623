"""Per-request confidence summary from the log-probabilities of the first generated tokens.

Over the first ``k`` generated tokens (default 32) it reports ``mean_top1`` (mean probability of the model's top-1
token), ``min_margin`` (smallest ``p(top-1) - p(top-2)``, in probability space) and ``low_frac`` (fraction of tokens whose
top-1 probability was below 0.5).  It is arithmetic over the top-k lists the sampler already produces for a request with
log-probabilities on; a request that asks for the summary without asking for log-probabilities gets them computed
internally (top-2) and not returned.

Reference parity: ``crates/spark-server/src/scheduler/conf_summary.rs`` (the three figures and the ``/metrics`` series
they feed; there the internal extraction is released after ``k`` tokens, here it stays on for the request).
"""
from __future__ import annotations

import math
from typing import List, Optional

DEFAULT_K = 32
INTERNAL_TOP = 2


def confidence_summary(entries: Optional[List[dict]], k: int = DEFAULT_K) -> Optional[dict]:
    """``entries``: the sampler's per-token records ``{"logprob": ..., "top": [(token id, logprob), ...]}``."""
    if not entries:
        return None
    p1s, margins = [], []
    for e in entries[:k]:
        top = sorted((float(lp) for _, lp in (e.get("top") or [])), reverse=True)
        if not top:
            top = [float(e.get("logprob", 0.0))]
        p1 = math.exp(top[0])
        p2 = math.exp(top[1]) if len(top) > 1 else 0.0
        p1s.append(p1)
        margins.append(p1 - p2)
    n = len(p1s)
    return {"tokens": n, "mean_top1": sum(p1s) / n, "min_margin": min(margins), "low_frac": sum(p < 0.5 for p in p1s) / n}
