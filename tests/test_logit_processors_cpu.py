"""The think / tool-call logit stages: each stage on hand-made rows, the stage order, and a request through the server
that must open a tool call right after its think block."""
import torch

from atlas_b200.server.logit_processors import ThinkToolPipeline, repeated_tool_call

OPEN, CLOSE, TOOL = 90, 91, 92
TEXT = {1: "the", 2: " ", 3: "p", 4: ".", 5: "ing", OPEN: "<think>", CLOSE: "</think>", TOOL: "<tool_call>"}


class _Seq:
    def __init__(self, out=()):
        self.output_tokens = list(out)


def _row(**hot):
    r = torch.zeros(100)
    for k, v in hot.items():
        r[int(k[1:])] = v
    return r


def _pipe(**kw):
    base = dict(think_open=[OPEN], think_close=[CLOSE], tool_open=[TOOL], token_text=lambda t: TEXT.get(t, "?"))
    base.update(kw)
    return ThinkToolPipeline(**base)


def test_close_tag_waits_for_a_word_boundary_and_never_returns():
    p = _pipe(starts_in_think=True)
    seq = _Seq([1])                                          # "...the": mid-word
    r = p(_row(t91=5.0), seq)
    assert r[CLOSE] == float("-inf") and p.stats.mid_word_defers == 1
    seq.output_tokens.append(2)                              # a space: the close tag is allowed again
    r = p(_row(t91=5.0), seq)
    assert r[CLOSE] == 5.0 and r[TOOL] == float("-inf")      # but no tool call inside thinking
    seq.output_tokens.append(CLOSE)
    r = p(_row(t91=5.0, t90=4.0, t92=1.0), seq)
    assert p.think_ended and not p.in_think
    assert r[CLOSE] == float("-inf") and r[OPEN] == float("-inf") and r[TOOL] == 1.0
    assert p.stats.post_close_masks == 1 and p.stats.tool_masks == 2


def test_required_tool_call_is_pinned_right_after_thinking_even_with_a_multi_token_opener():
    p = _pipe(starts_in_think=True, require_tool_call=True, tool_open=[7, 8])
    seq = _Seq([2, CLOSE])
    r = p(_row(t1=9.0), seq)
    assert int(r.argmax()) == 7 and int(torch.isfinite(r).sum()) == 1
    seq.output_tokens.append(7)
    r = p(_row(t1=9.0), seq)
    assert int(r.argmax()) == 8 and p.stats.pinned_tool_calls == 1
    seq.output_tokens.append(8)
    r = p(_row(t1=9.0), seq)
    assert p.tool_opened and int(r.argmax()) == 1            # free again once the opener is out
    # no pin without the requirement, and none once prose has started
    q = _pipe(starts_in_think=True)
    assert int(q(_row(t1=9.0), _Seq([2, CLOSE])).argmax()) == 1


def test_tool_call_loop_is_biased_not_masked():
    p = _pipe(suppress_tool_call=True)
    r = p(_row(t92=5.0, t1=0.0), _Seq([2]))
    assert r[TOOL] == 5.0 - 12.0 and p.stats.tool_biases == 1
    r = p(_row(t92=30.0), _Seq([2, 2]))
    assert int(r.argmax()) == TOOL                           # overwhelming evidence still wins
    msgs = [{"role": "user", "content": "x"}] + [
        {"role": "assistant", "tool_calls": [{"function": {"name": "ls", "arguments": "{\"p\": 1}"}}]},
        {"role": "tool", "content": "ok"}] * 3
    assert repeated_tool_call(msgs) and not repeated_tool_call(msgs[:-2])
    msgs[-2] = {"role": "assistant", "tool_calls": [{"function": {"name": "ls", "arguments": "{\"p\": 2}"}}]}
    assert not repeated_tool_call(msgs)


def test_confident_streak_ends_thinking_at_a_word_boundary():
    p = _pipe(starts_in_think=True, streak=3, min_think_tokens=2, think_close=[CLOSE, 4])
    seq = _Seq([2, 2])
    sure = lambda: _row(t1=20.0)
    for _ in range(2):
        p(sure(), seq)
        seq.output_tokens.append(1)
    assert not p.force_end_thinking and p.stats.early_think_ends == 0
    r = p(sure(), seq)                                       # third confident token, but "...the" is mid-word: armed, deferred
    assert p.force_end_thinking and int(r.argmax()) == 1
    seq.output_tokens.append(2)
    r = p(sure(), seq)
    assert int(r.argmax()) == CLOSE and int(torch.isfinite(r).sum()) == 1
    seq.output_tokens.append(CLOSE)
    r = p(sure(), seq)
    assert int(r.argmax()) == 4 and p.stats.early_think_ends == 1     # the rest of a multi-token close tag
    unsure = _pipe(starts_in_think=True, streak=3, min_think_tokens=0)
    for _ in range(5):
        unsure(_row(t1=0.5), _Seq([2]))
    assert not unsure.force_end_thinking


def test_margin_counter_reads_only_and_a_pinned_row_is_left_alone():
    p = _pipe(margin=True)
    a = _row(t1=3.0, t3=2.5)
    before = a.clone()
    p(a, _Seq([2]))
    assert torch.equal(a, before) and p.stats.low_margin == 1 and abs(p.stats.min_gap - 0.5) < 1e-6
    p(_row(t1=9.0), _Seq([2, 2]))
    assert p.stats.low_margin == 1 and p.stats.positions == 2
    pinned = torch.full((100,), float("-inf"))
    pinned[CLOSE] = 0.0
    q = _pipe(starts_in_think=True, guard_pinned=True)
    out = q(pinned.clone(), _Seq([1]))                       # mid-word, but another processor forced the close tag
    assert torch.equal(out, pinned)


def test_server_request_with_required_tool_call_opens_it_after_thinking():
    from atlas_b200.server.generation import GenRequest
    from tests.test_server_cpu import _client
    c, aeng, state = _client({"default_thinking": True, "tool_call_parser": "hermes"})
    try:
        from atlas_b200.server.generation import Generator
        gen = Generator(state)
        tools = [{"type": "function", "function": {"name": "ls", "parameters": {"type": "object", "properties": {}}}}]
        req = GenRequest(messages=[{"role": "user", "content": "hi"}], tools=tools, tool_choice="required", enable_thinking=True)
        procs = gen.prepare(req)[3]
        pipes = [p for p in procs if isinstance(p, ThinkToolPipeline)]
        assert len(pipes) == 1 and pipes[0].require_tool_call and pipes[0].tool and pipes[0].close
        plain = GenRequest(messages=[{"role": "user", "content": "hi"}], enable_thinking=False)
        assert not [p for p in gen.prepare(plain)[3] if isinstance(p, ThinkToolPipeline)]
    finally:
        aeng.shutdown(drain=False)
