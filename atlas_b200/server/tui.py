"""Terminal dashboard for a running server (``atlas_b200 tui --url http://host:port``).

The dashboard is a pure function of two polled snapshots: the Prometheus text of ``/metrics`` (parsed here, deltas
between polls give rates) and the JSON of ``/serve-config``.  Rendering produces plain text with ANSI colours, so it
works in any terminal and its output is testable as a string; when the terminal is not a TTY (or ``--plain``) one
status line per poll is printed instead, which keeps log scrapers working.

Sections: header (model, parallelism, uptime), load (active / waiting requests, KV occupancy bar), throughput
(tokens/s from counter deltas, requests/s, TTFT quantiles from the histogram), caches (prefix-cache hit rate,
speculative acceptance), health (GPU fault latch, preemptions) and a scrolling log of notable changes.

Reference parity: ``crates/spark-server/src/tui/`` (dashboard sections, plain-log mode as the compatibility path,
metrics deltas polled off the render thread).
"""
from __future__ import annotations

import json
import sys
import time
from typing import Dict, List, Optional, Tuple


def parse_prometheus(text: str) -> Dict[str, float]:
    """``name{labels}`` -> value for every sample line; label sets are kept verbatim in the key."""
    out: Dict[str, float] = {}
    for line in text.splitlines():
        if not line or line[0] == "#":
            continue
        try:
            key, val = line.rsplit(" ", 1)
            out[key] = float(val)
        except ValueError:
            continue
    return out


def _sum(m: Dict[str, float], prefix: str) -> float:
    return sum(v for k, v in m.items() if k == prefix or k.startswith(prefix + "{"))


def histogram_quantile(m: Dict[str, float], name: str, q: float) -> Optional[float]:
    """Quantile of a Prometheus histogram by linear interpolation inside the bucket (all label sets pooled)."""
    buckets: Dict[float, float] = {}
    for k, v in m.items():
        if k.startswith(name + "_bucket{") and 'le="' in k:
            le = k.split('le="', 1)[1].split('"', 1)[0]
            b = float("inf") if le == "+Inf" else float(le)
            buckets[b] = buckets.get(b, 0.0) + v
    if not buckets:
        return None
    edges = sorted(buckets)
    total = buckets[edges[-1]]
    if total <= 0:
        return None
    want, prev_c, prev_e = q * total, 0.0, 0.0
    for e in edges:
        c = buckets[e]
        if c >= want:
            if e == float("inf"):
                return prev_e
            frac = (want - prev_c) / max(c - prev_c, 1e-12)
            return prev_e + (e - prev_e) * frac
        prev_c, prev_e = c, e
    return edges[-2] if len(edges) > 1 else None


def bar(frac: float, width: int = 30) -> str:
    frac = max(0.0, min(1.0, frac))
    n = int(round(frac * width))
    return "[" + "#" * n + "." * (width - n) + f"] {100 * frac:5.1f}%"


class Dashboard:
    """Keeps the previous poll to turn counters into rates and to log notable transitions."""

    def __init__(self, colour: bool = True):
        self.prev: Optional[Tuple[float, Dict[str, float]]] = None
        self.t0 = time.monotonic()
        self.colour = colour
        self.log: List[str] = []

    def _c(self, s: str, code: str) -> str:
        return f"\x1b[{code}m{s}\x1b[0m" if self.colour else s

    def update(self, metrics_text: str, config: Optional[dict] = None, now: Optional[float] = None) -> str:
        now = time.monotonic() if now is None else now
        m = parse_prometheus(metrics_text)
        rates = {"tok_s": 0.0, "req_s": 0.0}
        if self.prev is not None:
            dt = max(1e-6, now - self.prev[0])
            pm = self.prev[1]
            rates["tok_s"] = max(0.0, _sum(m, "atlas_generation_tokens_total") - _sum(pm, "atlas_generation_tokens_total")) / dt
            rates["req_s"] = max(0.0, _sum(m, "atlas_requests_total") - _sum(pm, "atlas_requests_total")) / dt
            if m.get("atlas_gpu_fault", 0) and not pm.get("atlas_gpu_fault", 0):
                self.log.append(f"{now - self.t0:8.1f}s  GPU fault latched: the server answers 503 until it is restarted")
            dp = m.get("atlas_preemptions_total", 0) - pm.get("atlas_preemptions_total", 0)
            if dp > 0:
                self.log.append(f"{now - self.t0:8.1f}s  {int(dp)} sequence(s) preempted (KV pressure)")
        self.prev = (now, m)
        return self.render(m, rates, config or {}, now - self.t0)

    def render(self, m: Dict[str, float], rates: Dict[str, float], cfg: dict, uptime: float) -> str:
        total, free = m.get("atlas_kv_blocks_total", 0.0), m.get("atlas_kv_blocks_free", 0.0)
        used = (total - free) / total if total else 0.0
        look, hits = m.get("atlas_prefix_cache_lookups_total", 0.0), m.get("atlas_prefix_cache_hits_total", 0.0)
        prop, acc = m.get("atlas_spec_proposed_tokens_total", 0.0), m.get("atlas_spec_accepted_tokens_total", 0.0)
        q50 = histogram_quantile(m, "atlas_time_to_first_token_seconds", 0.5)
        q90 = histogram_quantile(m, "atlas_time_to_first_token_seconds", 0.9)
        fault = m.get("atlas_gpu_fault", 0.0) > 0
        ms = lambda v: "   n/a" if v is None else f"{v * 1e3:6.0f}"
        lines = [
            self._c(f" atlas_b200  {cfg.get('model', '?')}  tp={cfg.get('tp_size', 1)} ep={cfg.get('ep_size', 1)}  "
                    f"up {int(uptime) // 3600:02d}:{int(uptime) // 60 % 60:02d}:{int(uptime) % 60:02d}", "1;36"),
            f" load        active {int(m.get('atlas_requests_active', 0)):4d}   waiting {int(m.get('atlas_requests_waiting', 0)):4d}",
            f" kv cache    {bar(used)}  ({int(total - free)}/{int(total)} blocks)",
            f" throughput  {rates['tok_s']:9.1f} tok/s   {rates['req_s']:6.2f} req/s   "
            f"TTFT p50 {ms(q50)} ms  p90 {ms(q90)} ms",
            f" prefix      {bar(hits / look if look else 0.0, 20)}  hit tokens {int(m.get('atlas_prefix_cache_hit_tokens_total', 0))}",
            f" speculative {bar(acc / prop if prop else 0.0, 20)}  accepted {int(acc)}/{int(prop)}",
            " health      " + (self._c("GPU FAULT", "1;31") if fault else self._c("ok", "32")) +
            f"   preemptions {int(m.get('atlas_preemptions_total', 0))}",
        ]
        if self.log:
            lines.append(" events")
            lines += ["   " + l for l in self.log[-6:]]
        return "\n".join(lines)

    def status_line(self, metrics_text: str, now: Optional[float] = None) -> str:
        """The plain (non-TTY) form: one greppable line per poll."""
        self.update(metrics_text, None, now)
        m = self.prev[1]
        return (f"active={int(m.get('atlas_requests_active', 0))} waiting={int(m.get('atlas_requests_waiting', 0))} "
                f"kv_free={int(m.get('atlas_kv_blocks_free', 0))} gen_tokens={int(_sum(m, 'atlas_generation_tokens_total'))} "
                f"fault={int(m.get('atlas_gpu_fault', 0))}")


def run(url: str, interval: float = 1.0, plain: Optional[bool] = None, iterations: Optional[int] = None, fetch=None) -> int:
    """Poll ``url`` and redraw.  ``fetch(path) -> str`` can replace the HTTP client (tests)."""
    if fetch is None:
        import requests

        def fetch(path: str) -> str:
            return requests.get(url.rstrip("/") + path, timeout=5).text
    plain = (not sys.stdout.isatty()) if plain is None else plain
    dash = Dashboard(colour=not plain)
    cfg = None
    n = 0
    while iterations is None or n < iterations:
        try:
            text = fetch("/metrics")
            if cfg is None:
                try:
                    cfg = json.loads(fetch("/serve-config"))
                except Exception:
                    cfg = {}
            if plain:
                print(dash.status_line(text), flush=True)
            else:
                sys.stdout.write("\x1b[2J\x1b[H" + dash.update(text, cfg) + "\n")
                sys.stdout.flush()
        except KeyboardInterrupt:
            return 0
        except Exception as ex:
            print(f"[tui] {url}: {ex}", file=sys.stderr)
        n += 1
        if iterations is None or n < iterations:
            time.sleep(interval)
    return 0
