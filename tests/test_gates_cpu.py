"""Quality / isolation gates on CPU: contamination scoring (pure classifier + a run on a tiny engine, plus an engine
that is made to leak), function-call scoring, the agent loop over the fake workspace, and the serve matrix."""
import json

import pytest

from atlas_b200.bench import gates, ladder
from atlas_b200.config import EngineConfig, tiny_dense, tiny_hybrid
from atlas_b200.engine import LLMEngine
from atlas_b200.models import build_model


def _driver(mk=tiny_dense, **kw):
    eng = LLMEngine(build_model(mk()).init_random(0), EngineConfig(block_size=16, num_kv_blocks=256, max_num_seqs=8,
                                                                   max_prefill_tokens=64, **kw))
    return ladder.EngineDriver(eng)


def test_contamination_classifier_table():
    c = gates.classify
    ref, can, other = [1, 2, 3, 4, 5], [9, 9], [[9, 9], [7, 7, 7]]
    assert c(ref, ref, ref, can, other)[0] == "identical"
    assert c(ref, ref, [1, 2, 8, 4, 5], can, other) == ("diverged", 2)
    assert c(ref, [1, 2, 3, 4, 6], ref, can, other)[0] == "alone_unstable"
    assert c(ref, ref, [1, 7, 7, 7, 5], can, other)[0] == "contaminated"       # another request's canary in the reply
    assert c(ref, ref, [1, 9, 9, 4, 5], can, other)[0] == "diverged"           # its OWN canary is not leakage
    assert c(ref, ref, [1], can, other)[0] == "unmeasured"
    assert c(None, ref, ref, can, other)[0] == "unmeasured"


@pytest.mark.parametrize("mk", [tiny_dense, tiny_hybrid])
def test_contamination_gate_passes_on_the_engine(mk):
    res = gates.contamination_gate(_driver(mk, enable_prefix_caching=True), 1024, n_prompts=4, prompt_len=40, osl=10, rungs=(2, 4))
    assert res["pass"] and res["compared"] >= 8 and res["identical"] == res["compared"], res


def test_contamination_gate_catches_a_leaky_driver():
    inner = _driver()

    class Leaky:
        def run_batch(self, prompts, max_tokens, **kw):
            traces = inner.run_batch(prompts, max_tokens)
            if len(prompts) > 1:                              # under concurrency request 0 gets request 1's prompt head
                traces[0].tokens[2:8] = prompts[1][:6]
            return traces
    res = gates.contamination_gate(Leaky(), 1024, n_prompts=4, prompt_len=40, osl=12, rungs=(2,))
    assert not res["pass"] and res["contaminated"] >= 1


def test_function_call_scoring():
    exp = [{"name": "get_weather", "arguments": {"city": "Oslo", "days": {"any_of": [3, "3"]}}, "optional": ["units"]}]
    ok = gates.score_call
    assert ok([{"name": "get_weather", "arguments": {"city": "oslo ", "days": 3}}], exp)[0]
    assert ok([{"name": "get_weather", "arguments": json.dumps({"city": "Oslo", "days": "3", "units": "c"})}], exp)[0]
    assert not ok([{"name": "get_weather", "arguments": {"city": "Bergen", "days": 3}}], exp)[0]
    assert not ok([{"name": "get_weather", "arguments": {"city": "Oslo"}}], exp)[0]
    assert not ok([{"name": "get_weather", "arguments": {"city": "Oslo", "days": 3, "zip": 1}}], exp)[0]
    assert not ok([], exp)[0]
    cases = [{"category": "simple", "messages": [], "tools": [], "expected": exp},
             {"category": "irrelevance", "messages": [], "tools": [], "expected": []}]
    res = gates.function_call_gate(lambda m, t: [{"name": "get_weather", "arguments": {"city": "Oslo", "days": 3}}], cases, floor=0.4)
    assert res["overall"] == 0.5 and res["categories"] == {"simple": 1.0, "irrelevance": 0.0} and res["pass"]


def test_agentic_loop_over_fake_workspace():
    script = [
        [{"name": "write_file", "arguments": {"path": "src/main.rs", "content": "fn ping() -> &'static str { \"pong\" }"}}],
        [{"name": "run", "arguments": {"command": "cargo test"}}],
        [{"name": "run", "arguments": {"command": "cargo run --serve"}}],
        [{"name": "http_get", "arguments": {"path": "/ping"}}],
    ]

    def good(messages, tools):
        turn = sum(1 for m in messages if m["role"] == "assistant")
        return "working", script[min(turn, len(script) - 1)]
    res = gates.agentic_gate(good, iterations=2)
    assert res["pass"] and all(r["turns"] == 4 for r in res["rows"])
    lazy = gates.agentic_gate(lambda m, t: ("done", []), iterations=1)
    assert not lazy["pass"]


def test_serve_matrix_rows_and_identity_bar():
    class Handle:
        def __init__(self, name, lie=False):
            self.name, self.lie, self.d, self.max_context = name, lie, _driver(), 256

        def models(self):
            return ["something-else"] if self.lie else [self.name]

        def run_batch(self, prompts, max_tokens, **kw):
            return self.d.run_batch(prompts, max_tokens)

        def close(self):
            pass
    res = gates.serve_matrix(lambda n: Handle(n, lie=(n == "swapped")), ["tiny-a", "swapped"], baselines={"tiny-a": 0.001})
    rows = {r["model"]: r for r in res["rows"]}
    assert rows["tiny-a"]["verdict"] == "PASS" and rows["tiny-a"]["throughput"]["baseline"] == 0.001
    assert rows["swapped"]["verdict"] == "FAIL" and not rows["swapped"]["identity"]["pass"]
    assert rows["swapped"]["throughput"]["baseline"] == "no baseline"

    def broken(name):
        raise RuntimeError("no such checkpoint")
    assert gates.serve_matrix(broken, ["x"])["rows"][0]["verdict"] == "FAIL"
