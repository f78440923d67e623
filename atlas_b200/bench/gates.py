"""Quality / isolation gates that complement the speed gates of ``bench/ladder.py``.

* :func:`contamination_gate`  concurrent requests must not change each other's output.  Four legs: two solo reference
  passes (a prompt whose two solo runs differ is ``alone_unstable`` and is not blamed on concurrency), the concurrent
  rungs, and a solo post-check (a difference there is ``persistent``: state survived the concurrent episode).  Every
  prompt carries a canary token run that belongs to it alone; a foreign canary in a reply is leakage on its own evidence.
* :func:`function_call_gate`  single-turn function-calling accuracy over a list of cases, scored by an AST-style
  comparison of the parsed call (name, then every expected argument by value, extra arguments counted as errors).
* :func:`agentic_gate`        a bounded agent loop (model -> tool call -> tool result -> ...) over a scripted task with a
  pass predicate on the final tool state; tools are in-process fakes, nothing is executed on the host.
* :func:`serve_matrix`        boot every listed preset / checkpoint in turn, check that the model list names what was
  loaded, run coherence / tool-call / long-context / throughput probes, record one row each.

All of them take a *driver* with ``run_batch(prompts, max_tokens, ...) -> [RequestTrace]`` or a ``chat(messages, tools)``
callable, so they run in-process on CPU (tests) and over HTTP (``atlas_b200 benchmark``).

Reference parity: ``crates/avarok-plugin/src/benchmarks/{contamination,bfcl,agentic,serve_matrix}/``.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple


# ----------------------------------------------------------------------------------------------------- contamination
@dataclass
class ContaminationScore:
    prompts: int = 0
    rungs: int = 0
    compared: int = 0
    identical: int = 0
    diverged: int = 0
    contaminated: int = 0
    persistent: int = 0
    alone_unstable: int = 0
    unmeasured: int = 0
    details: List[dict] = field(default_factory=list)

    @property
    def passed(self) -> bool:
        return (self.compared > 0 and self.diverged == 0 and self.contaminated == 0 and self.persistent == 0
                and self.alone_unstable == 0)

    def as_dict(self) -> dict:
        d = {k: getattr(self, k) for k in ("prompts", "rungs", "compared", "identical", "diverged", "contaminated", "persistent",
                                           "alone_unstable", "unmeasured")}
        d["pass"] = self.passed
        d["details"] = self.details[:32]
        return d


def _common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


def classify(ref_a: Optional[Sequence[int]], ref_b: Optional[Sequence[int]], got: Optional[Sequence[int]], own_canary: Sequence[int],
             foreign_canaries: Sequence[Sequence[int]], min_tokens: int = 4) -> Tuple[str, int]:
    """Class of one prompt at one rung and the position of the first difference (pure function)."""
    if ref_a is None or ref_b is None or got is None or len(got) < min_tokens:
        return "unmeasured", 0
    if list(ref_a) != list(ref_b):
        return "alone_unstable", _common_prefix(ref_a, ref_b)
    gl = list(got)
    for c in foreign_canaries:
        c = list(c)
        if c and c != list(own_canary) and any(gl[i:i + len(c)] == c for i in range(len(gl) - len(c) + 1)):
            return "contaminated", 0
    if gl == list(ref_a):
        return "identical", len(gl)
    return "diverged", _common_prefix(gl, ref_a)


def contamination_gate(driver, vocab: int, n_prompts: int = 8, prompt_len: int = 48, osl: int = 24, rungs: Sequence[int] = (2, 4, 8),
                       seed: int = 11, canary_len: int = 6) -> dict:
    """Runs the four legs against ``driver`` (greedy, fixed seed) and scores them."""
    import torch
    g = torch.Generator().manual_seed(seed)
    canaries = [torch.randint(3, vocab, (canary_len,), generator=g).tolist() for _ in range(n_prompts)]
    prompts = []
    for i in range(n_prompts):
        body = torch.randint(3, vocab, (prompt_len - 2 * canary_len,), generator=g).tolist()
        prompts.append(canaries[i] + body + canaries[i])                # the canary frames the prompt

    def solo() -> List[Optional[List[int]]]:
        outs = []
        for p in prompts:
            try:
                outs.append(list(driver.run_batch([p], osl)[0].tokens))
            except Exception:
                outs.append(None)
        return outs
    for p in prompts:                                                   # prime: every leg runs cache-warm
        try:
            driver.run_batch([p], 1)
        except Exception:
            pass
    ref_a, ref_b = solo(), solo()
    score = ContaminationScore(prompts=n_prompts, rungs=len(rungs))
    for c in rungs:
        for lo in range(0, n_prompts, c):
            idx = list(range(lo, min(n_prompts, lo + c)))
            try:
                traces = driver.run_batch([prompts[i] for i in idx], osl)
                outs = [list(t.tokens) for t in traces]
            except Exception:
                outs = [None] * len(idx)
            for i, got in zip(idx, outs):
                cls, at = classify(ref_a[i], ref_b[i], got, canaries[i], canaries)
                _tally(score, cls, {"prompt": i, "rung": c, "class": cls, "at": at})
    post = solo()
    for i, got in enumerate(post):
        cls, at = classify(ref_a[i], ref_b[i], got, canaries[i], canaries)
        if cls == "diverged":
            cls = "persistent"
        if cls in ("persistent", "contaminated"):
            _tally(score, cls, {"prompt": i, "rung": "post", "class": cls, "at": at})
    return score.as_dict()


def _tally(score: ContaminationScore, cls: str, detail: dict) -> None:
    setattr(score, cls, getattr(score, cls) + 1)
    if cls in ("identical", "diverged", "contaminated", "persistent"):
        score.compared += 1
    if cls != "identical":
        score.details.append(detail)


# ----------------------------------------------------------------------------------------------------- function calling
def _values_equal(got: Any, want: Any) -> bool:
    if isinstance(want, float) or isinstance(got, float):
        try:
            return abs(float(got) - float(want)) <= 1e-6 * max(1.0, abs(float(want)))
        except (TypeError, ValueError):
            return False
    if isinstance(want, str) and isinstance(got, str):
        return got.strip().lower() == want.strip().lower()
    if isinstance(want, list) and isinstance(got, list):
        return len(want) == len(got) and all(_values_equal(a, b) for a, b in zip(got, want))
    if isinstance(want, dict) and isinstance(got, dict):
        return set(want) == set(got) and all(_values_equal(got[k], want[k]) for k in want)
    return got == want


def score_call(got_calls: List[dict], expected: List[dict]) -> Tuple[bool, str]:
    """AST-style check of one case: the same number of calls, and per call the same function name, every expected
    argument present with an equal value (an expected value may be a list of acceptable alternatives under the key
    ``"any_of"``), and no argument that was not expected."""
    if len(got_calls) != len(expected):
        return False, f"expected {len(expected)} call(s), got {len(got_calls)}"
    for g, e in zip(got_calls, expected):
        if g.get("name") != e.get("name"):
            return False, f"function {g.get('name')!r} != {e.get('name')!r}"
        ga = g.get("arguments", {})
        if isinstance(ga, str):
            try:
                ga = json.loads(ga or "{}")
            except ValueError:
                return False, "arguments are not JSON"
        for k, want in (e.get("arguments") or {}).items():
            if k not in ga:
                return False, f"missing argument {k!r}"
            alts = want["any_of"] if isinstance(want, dict) and "any_of" in want else [want]
            if not any(_values_equal(ga[k], w) for w in alts):
                return False, f"argument {k!r}: {ga[k]!r}"
        extra = set(ga) - set(e.get("arguments") or {}) - set(e.get("optional", []))
        if extra:
            return False, f"unexpected argument(s) {sorted(extra)}"
    return True, "ok"


def function_call_gate(chat: Callable[[List[dict], List[dict]], List[dict]], cases: List[dict], floor: Optional[float] = None) -> dict:
    """``chat(messages, tools) -> [{"name", "arguments"}]``; ``cases[i] = {"category", "messages", "tools", "expected"}``.
    Reports overall accuracy, the per-category accuracies and their unweighted mean (``normalized``)."""
    by_cat: Dict[str, List[bool]] = {}
    failures = []
    for i, c in enumerate(cases):
        try:
            got = chat(c["messages"], c.get("tools", []))
            ok, why = score_call(got, c.get("expected", []))
        except Exception as ex:                                         # a transport error is a miss, not a crash of the run
            ok, why = False, f"error: {ex}"
        by_cat.setdefault(c.get("category", "simple"), []).append(ok)
        if not ok:
            failures.append({"case": i, "why": why})
    n = sum(len(v) for v in by_cat.values())
    overall = sum(sum(v) for v in by_cat.values()) / max(1, n)
    cats = {k: sum(v) / len(v) for k, v in by_cat.items()}
    res = {"n": n, "overall": overall, "normalized": sum(cats.values()) / max(1, len(cats)), "categories": cats,
           "failures": failures[:32]}
    if floor is not None:
        res["pass"] = overall >= floor
    return res


# ----------------------------------------------------------------------------------------------------- agentic loop
class FakeWorkspace:
    """In-memory stand-in for the sandbox an agent works in: files, a command log, a 'server' that answers /ping once
    the agent has written a handler containing ``pong`` and asked to run it.  Nothing touches the host."""

    def __init__(self):
        self.files: Dict[str, str] = {}
        self.log: List[str] = []
        self.running = False

    TOOLS = [
        {"type": "function", "function": {"name": "write_file", "parameters": {"type": "object", "properties": {
            "path": {"type": "string"}, "content": {"type": "string"}}, "required": ["path", "content"]}}},
        {"type": "function", "function": {"name": "run", "parameters": {"type": "object", "properties": {
            "command": {"type": "string"}}, "required": ["command"]}}},
        {"type": "function", "function": {"name": "http_get", "parameters": {"type": "object", "properties": {
            "path": {"type": "string"}}, "required": ["path"]}}},
    ]

    def call(self, name: str, args: dict) -> str:
        self.log.append(f"{name}({json.dumps(args, sort_keys=True)[:120]})")
        if name == "write_file":
            self.files[str(args.get("path", ""))] = str(args.get("content", ""))
            return "written"
        if name == "run":
            cmd = str(args.get("command", ""))
            if "test" in cmd:
                return "tests passed" if any("pong" in v for v in self.files.values()) else "tests failed: no handler"
            if "serve" in cmd or "run" in cmd:
                self.running = any("pong" in v for v in self.files.values())
                return "listening" if self.running else "build failed"
            return "ok"
        if name == "http_get":
            return "pong" if (self.running and str(args.get("path", "")).rstrip("/").endswith("ping")) else "connection refused"
        return f"unknown tool {name}"

    def passed(self) -> bool:
        return self.running and any("http_get" in l and "ping" in l for l in self.log)


def agentic_gate(chat: Callable[[List[dict], List[dict]], Tuple[str, List[dict]]], iterations: int = 3, max_turns: int = 12,
                 task: str = "Create a web server with a /ping endpoint that answers pong, add a test, run the tests, "
                             "start the server and check /ping.") -> dict:
    """``chat(messages, tools) -> (text, [{"name", "arguments", "id"}])``.  One fresh workspace per iteration; an
    iteration passes when the workspace ends up serving ``/ping`` and the agent verified it."""
    rows = []
    for it in range(iterations):
        ws = FakeWorkspace()
        msgs = [{"role": "system", "content": "You are a coding agent. Use the tools."}, {"role": "user", "content": task}]
        t0 = time.perf_counter()
        turns = 0
        for turns in range(1, max_turns + 1):
            try:
                text, calls = chat(msgs, FakeWorkspace.TOOLS)
            except Exception as ex:
                msgs.append({"role": "assistant", "content": f"error: {ex}"})
                break
            msgs.append({"role": "assistant", "content": text, "tool_calls": [
                {"id": c.get("id", f"call_{turns}_{j}"), "type": "function",
                 "function": {"name": c["name"], "arguments": json.dumps(c.get("arguments", {}))}} for j, c in enumerate(calls)]})
            if not calls:
                break
            for j, c in enumerate(calls):
                args = c.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args or "{}")
                    except ValueError:
                        args = {}
                msgs.append({"role": "tool", "tool_call_id": c.get("id", f"call_{turns}_{j}"), "content": ws.call(c["name"], args)})
            if ws.passed():
                break
        rows.append({"iteration": it, "pass": ws.passed(), "turns": turns, "seconds": time.perf_counter() - t0,
                     "tool_calls": len(ws.log)})
    ok = sum(r["pass"] for r in rows)
    return {"iterations": iterations, "passed": ok, "pass": ok == iterations, "total_seconds": sum(r["seconds"] for r in rows),
            "rows": rows}


# ----------------------------------------------------------------------------------------------------- serve matrix
def serve_matrix(boot: Callable[[str], Any], rounds: Sequence[str], probes: Optional[Dict[str, Callable[[Any], dict]]] = None,
                 baselines: Optional[Dict[str, float]] = None) -> dict:
    """``boot(name)`` returns a handle with ``models() -> [str]`` (what the endpoint lists), ``run_batch`` and
    ``close()``.  A round is READY only when the model list names the checkpoint that was asked for; every probe
    returns ``{"pass": bool, ...}``.  The throughput bar is compared with ``baselines[name]`` and says "no baseline"
    where there is none instead of passing silently."""
    probes = probes or DEFAULT_PROBES
    rows = []
    for name in rounds:
        row: Dict[str, Any] = {"model": name}
        h = None
        try:
            t0 = time.perf_counter()
            h = boot(name)
            row["boot_s"] = time.perf_counter() - t0
            listed = list(h.models())
            row["identity"] = {"pass": name in listed, "listed": listed}
            for pname, fn in probes.items():
                try:
                    row[pname] = fn(h)
                except Exception as ex:
                    row[pname] = {"pass": False, "error": str(ex)[:200]}
            tps = (row.get("throughput") or {}).get("tok_s")
            if tps is not None:
                base = (baselines or {}).get(name)
                row["throughput"]["baseline"] = base if base is not None else "no baseline"
                if base is not None:
                    row["throughput"]["pass"] = tps >= 0.9 * base
        except Exception as ex:
            row["boot_error"] = str(ex)[:300]
        finally:
            if h is not None and hasattr(h, "close"):
                h.close()
        bars = [v.get("pass") for k, v in row.items() if isinstance(v, dict) and "pass" in v]
        row["verdict"] = "PASS" if bars and all(bars) and "boot_error" not in row else "FAIL"
        rows.append(row)
    return {"rounds": len(rows), "passed": sum(r["verdict"] == "PASS" for r in rows), "rows": rows}


def _probe_coherence(h) -> dict:
    """Greedy decoding twice gives the same tokens, and the output is not one token repeated."""
    p = list(range(5, 37))
    a = list(h.run_batch([p], 16)[0].tokens)
    b = list(h.run_batch([p], 16)[0].tokens)
    return {"pass": a == b and len(a) >= 8, "deterministic": a == b, "tokens": len(a), "distinct": len(set(a))}


def _probe_long_context(h) -> dict:
    n = min(getattr(h, "max_context", 512) // 2, 2048)
    tr = h.run_batch([[(7 * i) % 997 + 3 for i in range(n)]], 4)[0]
    return {"pass": len(tr.tokens) >= 1, "prompt_tokens": n, "ttft_ms": None if tr.ttft is None else tr.ttft * 1e3}


def _probe_throughput(h) -> dict:
    t0 = time.perf_counter()
    traces = h.run_batch([[3 + (i * 13 + j) % 500 for j in range(32)] for i in range(4)], 32)
    dt = time.perf_counter() - t0
    n = sum(len(t.tokens) for t in traces)
    return {"pass": n > 0, "tok_s": n / dt if dt > 0 else 0.0}


DEFAULT_PROBES: Dict[str, Callable[[Any], dict]] = {"coherence": _probe_coherence, "long_context": _probe_long_context,
                                                    "throughput": _probe_throughput}
