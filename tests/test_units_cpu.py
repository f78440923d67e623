"""Unit tier (CPU): tool-call parsers, reasoning splitter, grammar matcher, block pool + radix cache (incl. a
randomised model check), scheduler behaviours (chunked prefill, preemption with resume, admission), sampler
distributions and penalties, collective protocol with injected failures, fault latch classification."""
import json
import random

import pytest
import torch

from atlas_b200.config import EngineConfig, tiny_dense
from atlas_b200.engine import LLMEngine
from atlas_b200.kv import BlockPool, RadixCache
from atlas_b200.kv.block_manager import OutOfBlocks
from atlas_b200.models import build_model
from atlas_b200.ops import reference as ref
from atlas_b200.parallel.comm import CommError, FakeWorld
from atlas_b200.sampling import RequestRng, SamplingParams
from atlas_b200.sched import FinishReason, SeqStatus
from atlas_b200.server.reasoning import ReasoningSplitter, split_reasoning
from atlas_b200.server.tool_parsers import StreamingToolParser, default_parser_for, get_parser
from atlas_b200.utils.fault import Fatality, FaultLatch, classify_probe

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}, "metric": {"type": "boolean"}}}}}]


# ----------------------------------------------------------------------------------------------------- tool parsers
@pytest.mark.parametrize("name,text", [
    ("hermes", 'Sure.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo", "days": 3}}\n</tool_call>'),
    ("qwen3_coder", "Sure.<tool_call>\n<function=get_weather>\n<parameter=city>\nOslo\n</parameter>\n<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>"),
    ("mistral", 'Sure.[TOOL_CALLS][{"name": "get_weather", "arguments": {"city": "Oslo", "days": 3}}]'),
    ("minimax_xml", 'Sure.<minimax:tool_call>\n<invoke name="get_weather">\n<parameter name="city">Oslo</parameter>\n<parameter name="days">3</parameter>\n</invoke>\n</minimax:tool_call>'),
    ("gemma", 'Sure.\n```tool_code\nget_weather(city="Oslo", days=3)\n```'),
    ("lfm3", "Sure.<tool_call>\n<function=get_weather>\n<parameter=city>\nOslo\n</parameter>\n<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>"),
    ("poolside_v1", "Sure.<tool_call>get_weather<arg_key>city</arg_key><arg_value>Oslo</arg_value><arg_key>days</arg_key><arg_value>3</arg_value></tool_call>"),
])
def test_tool_parsers_extract_calls(name, text):
    content, calls = get_parser(name, TOOLS).parse(text)
    assert len(calls) == 1 and calls[0].name == "get_weather"
    args = json.loads(calls[0].arguments)
    assert args["city"] == "Oslo" and args["days"] == 3          # typed through the declared schema
    assert "Sure." in content and "get_weather" not in content
    oa = calls[0].to_openai(0)
    assert oa["type"] == "function" and oa["function"]["name"] == "get_weather" and oa["id"]


def test_bare_json_and_plain_text_and_defaults():
    p = get_parser("bare_json", TOOLS)
    _, calls = p.parse('{"name": "get_weather", "arguments": {"city": "Rome"}}')
    assert calls and json.loads(calls[0].arguments) == {"city": "Rome"}
    for name in ("hermes", "qwen3_coder", "mistral", "bare_json", "gemma"):
        content, calls = get_parser(name, TOOLS).parse("just words, no call")
        assert calls == [] and content == "just words, no call"
    assert default_parser_for("qwen3_next") == "qwen3_coder" and default_parser_for("mistral") == "mistral"
    assert default_parser_for("qwen3_moe") == "hermes"
    with pytest.raises(ValueError):
        get_parser("nope")


def test_streaming_tool_parser_holds_back_markers():
    text = 'Let me check. <tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo"}}\n</tool_call>'
    for step in (1, 3, 7, 1000):
        sp = StreamingToolParser(get_parser("hermes", TOOLS))
        shown = "".join(sp.push(text[i:i + step]) for i in range(0, len(text), step))
        rest, calls = sp.finish()
        assert "<" not in shown and shown.startswith("Let me check.")
        assert len(calls) == 1 and calls[0].name == "get_weather"
    sp = StreamingToolParser(get_parser("hermes", TOOLS))
    shown = "".join(sp.push(ch) for ch in "a < b and <tool is not a call")
    rest, calls = sp.finish()
    assert calls == [] and shown + rest == "a < b and <tool is not a call"


# ----------------------------------------------------------------------------------------------------- reasoning
def test_reasoning_splitter_any_chunking():
    text = "<think>\nstep one\nstep two</think>\n\nThe answer is 4."
    for step in (1, 2, 5, 100):
        sp = ReasoningSplitter()
        r = c = ""
        for i in range(0, len(text), step):
            a, b = sp.push(text[i:i + step])
            r, c = r + a, c + b
        a, b = sp.finish()
        r, c = r + a, c + b
        assert r.strip() == "step one\nstep two" and c == "The answer is 4."
    assert split_reasoning("no thinking here") == (None, "no thinking here")
    assert split_reasoning("already inside</think>done", starts_in_reasoning=True) == ("already inside", "done")
    r, c = split_reasoning("<think>never closed")
    assert r == "never closed" and c == ""


# ----------------------------------------------------------------------------------------------------- grammar
def test_byte_json_matcher_keeps_brackets_balanced():
    """The built-in fallback matcher (used when xgrammar is missing) works on byte-tokenizer ids (3 + byte): the
    output must open with an object, brackets close in order, string contents are free, then only EOS."""
    from atlas_b200.server.grammar import _ByteJsonMatcher
    good = '{"a": [1, 2.5, true, null], "b": {"c": "x\\"y}]"}}'
    m = _ByteJsonMatcher(1024)
    assert not bool(m.token_mask(1024)[3 + ord("x")]) and bool(m.token_mask(1024)[3 + ord("{")])
    for ch in good.encode():
        assert bool(m.token_mask(1024)[3 + ch]), f"byte {chr(ch)!r} should be allowed"
        assert m.accept(3 + ch)
    assert m.terminated()
    mask = m.token_mask(1024)
    assert bool(mask[2]) and int(mask.sum()) == 1                  # closed: EOS only
    m = _ByteJsonMatcher(1024)
    for ch in b'{"a": [1':
        m.accept(3 + ch)
    mask = m.token_mask(1024)
    assert bool(mask[3 + ord("]")]) and not bool(mask[3 + ord("}")])   # the array has to close first
    assert not m.accept(3 + ord("}"))


# ----------------------------------------------------------------------------------------------------- block pool / radix
def test_block_pool_refcounts():
    p = BlockPool(8, 16)
    a = p.alloc(3)
    p.inc_ref(a[:1])
    assert p.free(a) == 2 and p.ref_count(a[0]) == 1 and p.num_free == 7
    p.free(a[:1])
    p.check_invariants()
    with pytest.raises(ValueError):
        p.free(a[:1])
    with pytest.raises(OutOfBlocks):
        p.alloc(9)
    assert p.blocks_for_tokens(17) == 2 and p.high_water == 3


def test_radix_match_insert_evict():
    pool = BlockPool(16, 4)
    rc = RadixCache(pool)
    toks = list(range(13))
    blocks = pool.alloc(4)
    rc.insert(toks, blocks)                       # 3 full blocks published
    pool.free(blocks)                             # the sequence lets go; the tree keeps 3
    assert pool.num_used == 3
    m = rc.match(toks[:9] + [99, 98, 97])
    assert m.num_tokens == 8 and m.blocks == blocks[:2]
    m1 = rc.match(toks[:8])
    assert m1.num_tokens == 4                     # always leaves one token to compute
    rc.release(m1.nodes)
    pool.free(m1.blocks)
    assert rc.evict(10) == 1                      # only the unpinned leaf can go
    rc.release(m.nodes)
    pool.free(m.blocks)
    m2 = rc.match(toks[:8], namespace="other")
    assert m2.num_tokens == 0                     # namespaces (adapters / tenants) do not share
    assert rc.evict(10) == 2 and pool.num_used == 0
    pool.check_invariants()


def test_radix_randomised_against_model():
    """Random inserts / matches / evictions against a dict-of-prefixes model; references must balance."""
    rnd = random.Random(0)
    pool = BlockPool(64, 2)
    rc = RadixCache(pool)
    known = set()
    for _ in range(300):
        op = rnd.random()
        toks = [rnd.randrange(3) for _ in range(rnd.randrange(2, 12))]
        if op < 0.5:
            n = pool.blocks_for_tokens(len(toks))
            if pool.num_free < n:
                rc.evict(n)
            if pool.num_free < n:
                continue
            blocks = pool.alloc(n)
            rc.insert(toks, blocks)
            pool.free(blocks)
            for j in range(1, len(toks) // 2 + 1):
                known.add(tuple(toks[:2 * j]))
        elif op < 0.9:
            m = rc.match(toks)
            want = 0
            for j in range(1, (len(toks) - 1) // 2 + 1):
                if tuple(toks[:2 * j]) in known:
                    want = 2 * j
                else:
                    break
            assert m.num_tokens <= want            # evictions may have shortened it, never lengthened
            rc.release(m.nodes)
            pool.free(m.blocks)
        else:
            rc.evict(rnd.randrange(1, 6))
            known = {k for k in known if rc.match(list(k) + [0]).num_tokens == len(k) or True}
        pool.check_invariants()
    # drop every outstanding match reference taken inside the comprehension above, then clear
    rc.clear()
    assert pool.num_used >= 0


# ----------------------------------------------------------------------------------------------------- scheduler
def _engine(**kw):
    cfg = dict(block_size=16, num_kv_blocks=64, max_num_seqs=8, max_prefill_tokens=48)
    cfg.update(kw)
    return LLMEngine(build_model(tiny_dense()).init_random(0), EngineConfig(**cfg))


def _prompts(n, length, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def test_chunked_prefill_and_mixed_steps():
    eng = _engine(max_prefill_tokens=32)
    ids = [eng.add_request(p, SamplingParams(max_tokens=6, ignore_eos=True)) for p in _prompts(2, 80)]
    kinds = []
    while eng.has_unfinished():
        before = eng.stats.steps
        eng.step()
        assert eng.stats.steps == before + 1
        kinds.append(eng.scheduler.snapshot())
    assert eng.stats.prefill_tokens >= 160 and eng.stats.steps >= 160 // 32
    eng.pool.check_invariants()


def test_preemption_resumes_and_matches_uncontended_run():
    prompts = _prompts(4, 40)
    sp = SamplingParams(max_tokens=40, ignore_eos=True)
    want = [o.output_tokens for o in _engine(num_kv_blocks=64).generate(prompts, sp)]
    tight = _engine(num_kv_blocks=14, enable_prefix_caching=True)        # 4 x 80 tokens do not fit in 14 blocks
    got = [o.output_tokens for o in tight.generate(prompts, sp)]
    assert got == want
    assert tight.scheduler.num_preemptions > 0
    tight.pool.check_invariants()


def test_prefill_budget_not_a_block_multiple_cannot_livelock():
    """A long and a short prompt share a pool that holds the long one with little to spare and the per-step prefill
    budget is not a multiple of the block size: the second prompt must not be admitted on blocks the first still
    needs, and if prefills ever hold every block without one of them being able to advance, one yields."""
    from atlas_b200.sched import Scheduler
    from atlas_b200.sched.sequence import Sequence
    cfg = EngineConfig(block_size=16, num_kv_blocks=200, max_num_seqs=8, max_prefill_tokens=1000, max_seq_len=4096,
                       admission_watermark_tokens=0)
    pool = BlockPool(200, 16)
    sch = Scheduler(cfg, pool)
    a = Sequence("a", list(range(3180)), SamplingParams(max_tokens=1, ignore_eos=True))
    b = Sequence("b", list(range(100)), SamplingParams(max_tokens=1, ignore_eos=True))
    sch.add(a)
    sch.add(b)
    idle = 0
    for _ in range(64):
        out = sch.schedule()
        if not out.items:
            idle += 1
            assert idle < 3, "scheduler makes no progress"
            continue
        idle = 0
        for it in out.items:
            sch.on_chunk_computed(it)
            if it.seq.num_computed >= it.seq.num_tokens:
                sch.finish(it.seq, FinishReason.LENGTH)
        if not sch.has_work():
            break
    assert not sch.has_work()
    pool.check_invariants()

    # forced form of the same state: two partly allocated prefills hold every block
    pool2 = BlockPool(8, 16)
    sch2 = Scheduler(EngineConfig(block_size=16, num_kv_blocks=8, max_num_seqs=8, max_prefill_tokens=64,
                                  max_seq_len=4096), pool2)
    x = Sequence("x", list(range(100)), SamplingParams(max_tokens=1, ignore_eos=True))
    y = Sequence("y", list(range(100)), SamplingParams(max_tokens=1, ignore_eos=True))
    for s_ in (x, y):
        s_.status = SeqStatus.PREFILL
        s_.blocks = pool2.alloc(4)
        s_.num_computed = 64
        sch2.prefilling.append(s_)
    out = sch2.schedule()
    assert out.items and out.items[0].seq is x and y in sch2.waiting


def test_admission_and_rejection():
    from atlas_b200.engine import RequestRejected
    eng = _engine(num_kv_blocks=8, max_seq_len=256)
    with pytest.raises(RequestRejected):
        eng.add_request([], SamplingParams())
    with pytest.raises(RequestRejected):
        eng.add_request([5000], SamplingParams())
    with pytest.raises(RequestRejected):
        eng.add_request([1] * 300, SamplingParams())
    rid = eng.add_request([1] * 20, SamplingParams(max_tokens=1000))
    assert eng._seqs[rid].sampling.max_tokens == 256 - 20            # clamped to the context window
    assert eng.abort(rid) and not eng.has_unfinished() and eng.pool.num_free == 8


# ----------------------------------------------------------------------------------------------------- sampler
def _draw(logits, u, t=1.0, k=0, p=1.0, mp=0.0):
    return int(ref.sample(logits, torch.tensor([t]), torch.tensor([k]), torch.tensor([p]), torch.tensor([mp]),
                          torch.tensor([u])))


def test_sampler_distribution_and_filters():
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, -50.0]])
    p = torch.softmax(logits[0], -1)
    counts = torch.zeros(5)
    rng = RequestRng(7)
    for i in range(4000):
        counts[_draw(logits, rng.uniform(i))] += 1
    assert torch.allclose(counts / 4000, p, atol=0.03)
    rng = RequestRng(9)
    for i in range(200):                              # top-k 2 never leaves the two best; top-p / min-p 0.5 keep only the best
        u = rng.uniform(i)
        assert _draw(logits, u, k=2) in (0, 1)
        assert _draw(logits, u, p=0.5) == 0
        assert _draw(logits, u, mp=0.5) == 0
        assert _draw(logits, u, t=0.0) == 0
    assert int(ref.argmax_first(torch.tensor([[1.0, 3.0, 3.0]]))) == 1            # first index wins ties


def test_penalties_and_rng_is_position_addressed():
    logits = torch.tensor([[1.0, 1.0, -1.0, 1.0, 1.0, 1.0]])
    counts = torch.tensor([[0, 2, 1, 0, 0, 0]])
    prompt = torch.tensor([[False, False, False, True, False, False]])
    out = ref.apply_penalties(logits, counts, prompt, torch.tensor([2.0]), torch.tensor([0.5]), torch.tensor([0.25]))
    assert out[0, 0] == 1.0                                                   # unseen: untouched
    assert out[0, 1] == pytest.approx(1.0 / 2 - 0.25 * 2 - 0.5)               # generated twice
    assert out[0, 2] == pytest.approx(-1.0 * 2 - 0.25 - 0.5)                  # negative logits are multiplied
    assert out[0, 3] == pytest.approx(1.0 / 2)                                # prompt-only: repetition penalty only
    r = RequestRng(123)
    a = [r.uniform(i) for i in range(5)]
    assert a == [RequestRng(123).uniform(i) for i in range(5)] and len(set(a)) == 5
    assert all(0.0 <= x < 1.0 for x in a)
    assert RequestRng(None, "req-a").uniform(0) != RequestRng(None, "req-b").uniform(0)


# ----------------------------------------------------------------------------------------------------- comm / fault
def test_fake_collectives_and_injected_failures():
    w = FakeWorld(3, timeout_s=5.0)
    outs = w.run(lambda r: (w_comm := w.comm(r)).all_reduce(torch.full((4,), float(r + 1))).tolist()
                 + w_comm.all_gather(torch.tensor([r])).tolist())
    assert all(o == [6.0] * 4 + [0, 1, 2] for o in outs)
    # a rank that never joins: the others time out, get an error (not a hang) and their communicator is poisoned
    w = FakeWorld(3, timeout_s=0.2)
    w.dead.add(2)
    comms = [w.comm(r) for r in range(3)]

    def body(r):
        try:
            comms[r].all_reduce(torch.ones(2))
            return "ok"
        except CommError as e:
            return str(e)
    res = w.run(body)
    assert all("missing ranks [2]" in res[r] for r in (0, 1))
    assert comms[0].unhealthy and comms[1].unhealthy
    with pytest.raises(CommError):
        comms[0].barrier()                 # poisoned: fails fast from now on
    # a dropped contribution (lost message) is detected the same way
    w = FakeWorld(2, timeout_s=0.2)
    w.dropped.add((1, 1))
    res = w.run(lambda r: body_drop(w, r))
    assert "timed out" in res[0]


def body_drop(w, r):
    try:
        w.comm(r).all_reduce(torch.ones(1))
        return "ok"
    except CommError as e:
        return str(e)


def test_fault_latch_classification():
    assert classify_probe(False, True) is Fatality.NONE
    assert classify_probe(True, True) is Fatality.REQUEST_SCOPED
    assert classify_probe(True, False) is Fatality.CONTEXT_LOST
    latch = FaultLatch(probe=lambda: False)
    assert latch.observe_exception(ValueError("bad request")) is Fatality.REQUEST_SCOPED and not latch.tripped
    assert latch.observe_exception(RuntimeError("CUDA error: an illegal memory access was encountered")) is Fatality.CONTEXT_LOST
    assert latch.tripped and "illegal memory access" in latch.reason
    latch.trip("second reason")
    assert "illegal memory access" in latch.reason            # one-shot: the first reason sticks
    ok = FaultLatch(probe=lambda: True)
    assert ok.observe_exception(RuntimeError("CUDA error: out of memory")) is Fatality.REQUEST_SCOPED and not ok.tripped
    assert ok.observe_status_word(0x1234) is Fatality.REQUEST_SCOPED and ok.request_scoped_failures == 2


@pytest.mark.parametrize("hybrid", [False, True])
def test_host_tier_swaps_instead_of_recomputing(hybrid):
    """With swap space, a preempted decode parks its KV (and recurrent state) in host memory and resumes without
    recomputing its context: same tokens as an uncontended run, fewer prefill tokens than the recompute path."""
    from atlas_b200.config import tiny_hybrid
    mk = tiny_hybrid if hybrid else tiny_dense
    prompts = _prompts(4, 40)
    sp = SamplingParams(max_tokens=40, ignore_eos=True)

    def eng(**kw):
        return LLMEngine(build_model(mk()).init_random(0), EngineConfig(block_size=16, max_num_seqs=8, max_prefill_tokens=64, **kw))

    want = [o.output_tokens for o in eng(num_kv_blocks=64).generate(prompts, sp)]
    recompute = eng(num_kv_blocks=14)
    assert [o.output_tokens for o in recompute.generate(prompts, sp)] == want
    swap = eng(num_kv_blocks=14, swap_space_gb=0.01)
    assert swap.host_tier is not None and swap.host_tier.num_blocks >= 8
    got = [o.output_tokens for o in swap.generate(prompts, sp)]
    assert got == want
    assert swap.scheduler.num_swaps > 0 and swap.host_tier.blocks_in == swap.host_tier.blocks_out > 0
    assert swap.stats.prefill_tokens < recompute.stats.prefill_tokens
    assert swap.host_tier.num_free == swap.host_tier.num_blocks and not swap.scheduler.swapped
    swap.pool.check_invariants()


def test_disk_tier_below_host_tier(tmp_path):
    """A host tier too small for all parked sequences spills the ones that resume last to a swap file and brings them
    back through host blocks; tokens match the uncontended run and every tier ends empty."""
    prompts = _prompts(6, 40)
    sp = SamplingParams(max_tokens=40, ignore_eos=True)

    def eng(**kw):
        return LLMEngine(build_model(tiny_dense()).init_random(0), EngineConfig(block_size=16, max_num_seqs=8, max_prefill_tokens=64, **kw))

    want = [o.output_tokens for o in eng(num_kv_blocks=96).generate(prompts, sp)]
    e = eng(num_kv_blocks=14, swap_space_gb=0.01, disk_swap_gb=0.01, disk_swap_path=str(tmp_path))
    per_block = e.host_tier.record_bytes
    e.host_tier._free = e.host_tier._free[:6]                 # shrink the host tier to six blocks: one parked sequence
    e.host_tier.num_blocks = 6
    got = [o.output_tokens for o in e.generate(prompts, sp)]
    assert got == want
    disk = e.host_tier.disk
    assert disk is not None and disk.record_bytes == per_block
    assert e.scheduler.num_spills > 0 and disk.records_out == disk.records_in > 0
    assert disk.num_free == disk.num_records and e.host_tier.num_free == 6 and not e.scheduler.swapped
    e.pool.check_invariants()
    path = disk.path
    disk.close()
    import os
    assert not os.path.exists(path)


def test_loop_detector_and_engine_stop():
    from atlas_b200.server.loop_detector import LoopDetector
    det = LoopDetector(span=32, max_period=8, min_repeats=4, stride=1)
    g = torch.Generator().manual_seed(0)
    rnd = torch.randint(0, 1000, (200,), generator=g).tolist()
    assert det.check(rnd) is None
    assert det.check(rnd + [7, 8, 9] * 10) is None                  # 30 periodic tokens < span
    assert det.check(rnd + [7, 8, 9] * 11) == 3
    assert det.check(rnd + [5] * 32) == 1
    assert det.check([1, 2] * 8) is None                            # shorter than the span
    long_p = list(range(10))
    assert LoopDetector(span=32, max_period=8, min_repeats=4).check(rnd + long_p * 8) is None     # period 10 > max_period
    assert LoopDetector(span=32, max_period=16, min_repeats=4).check(rnd + long_p * 8) == 10

    # engine: a checker that fires ends the request with reason "stop" before max_tokens
    eng = _engine(num_kv_blocks=64)
    fired = LoopDetector(span=8, max_period=4, min_repeats=2, stride=1)

    class Forced:                              # make the model emit a cycle: every row is forced to token (n % 2)
        def __call__(self, row, seq):
            row = torch.full_like(row, float("-inf"))
            row[seq.num_output_tokens % 2] = 0.0
            return row
    rid = eng.add_request(_prompts(1, 12)[0], SamplingParams(max_tokens=64, ignore_eos=True), logits_processors=[Forced()],
                          stop_checker=fired)
    outs = {}
    while eng.has_unfinished():
        for o in eng.step():
            outs[o.request_id] = o
    assert outs[rid].finish_reason == "stop" and fired.period == 2
    assert 8 <= len(outs[rid].output_tokens) < 64


def test_context_compaction_stages():
    from atlas_b200.server.compaction import compact_messages
    count = lambda msgs: sum(len(str(m.get("content") or "")) // 4 + 4 for m in msgs)      # ~4 characters per token
    sys_m = {"role": "system", "content": "You are terse."}
    big_tool = {"role": "tool", "tool_call_id": "a", "content": "x" * 20000}
    chat = [sys_m,
            {"role": "user", "content": "list the files"},
            {"role": "assistant", "content": "", "tool_calls": [{"id": "a", "type": "function", "function": {"name": "ls", "arguments": "{}"}}]},
            big_tool,
            {"role": "assistant", "content": "done " * 200},
            {"role": "user", "content": "q" * 8000},
            {"role": "assistant", "content": "ok"},
            {"role": "user", "content": "and now?"},
            {"role": "assistant", "content": "sure"},
            {"role": "user", "content": "last question"}]
    same, rep = compact_messages(chat, count, budget=100000)
    assert same == chat and rep["stage"] == 0
    out, rep = compact_messages(chat, count, budget=4000)           # eliding the tool result is enough
    assert rep["stage"] == 1 and rep["elided"] == 1 and rep["dropped"] == 0 and count(out) <= 4000
    assert "elided" in out[3]["content"] and out[3]["content"].startswith("x") and len(out) == len(chat)
    assert chat[3]["content"] == "x" * 20000                        # the caller's list is untouched
    out, rep = compact_messages(chat, count, budget=1200)           # user turn has to shrink too
    assert rep["stage"] == 2 and count(out) <= 1200
    out, rep = compact_messages(chat, count, budget=150)            # old turns are dropped, tool result with its call
    assert rep["stage"] == 3 and rep["dropped"] >= 4
    assert out[0] == sys_m and out[1]["role"] == "system" and "left out" in out[1]["content"]
    assert [m["content"] for m in out[-4:]] == [m["content"] for m in chat[-4:]]
    assert not any(m.get("role") == "tool" for m in out)


def test_model_resolver_offline(tmp_path, monkeypatch):
    from atlas_b200.utils.model_resolver import ModelNotFound, resolve_model
    import os, time
    local = tmp_path / "ckpt"
    local.mkdir()
    (local / "config.json").write_text("{}")
    assert resolve_model(str(local)) == str(local)
    assert resolve_model("preset:tiny-dense") == "preset:tiny-dense"
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(ModelNotFound):
        resolve_model(str(empty))
    # search directories
    models = tmp_path / "models"
    (models / "Llama-X").mkdir(parents=True)
    (models / "Llama-X" / "config.json").write_text("{}")
    monkeypatch.setenv("ATLAS_MODEL_DIRS", str(models))
    assert resolve_model("meta/Llama-X") == str(models / "Llama-X")
    # hub cache: refs/main wins, else the newest snapshot with a config
    cache = tmp_path / "hf" / "hub"
    snaps = cache / "models--org--name" / "snapshots"
    for rev in ("aaa", "bbb"):
        (snaps / rev).mkdir(parents=True)
        (snaps / rev / "config.json").write_text("{}")
        time.sleep(0.02)
    monkeypatch.setenv("HF_HOME", str(tmp_path / "hf"))
    monkeypatch.delenv("HF_HUB_CACHE", raising=False)
    assert resolve_model("org/name") == str(snaps / "bbb")
    refs = cache / "models--org--name" / "refs"
    refs.mkdir()
    (refs / "main").write_text("aaa\n")
    assert resolve_model("org/name") == str(snaps / "aaa")
    assert resolve_model("org/name", revision="bbb") == str(snaps / "bbb")
    with pytest.raises(ModelNotFound) as ei:
        resolve_model("org/other")
    assert "models--org--other" in str(ei.value)


def test_output_sanitizer_stops():
    from atlas_b200.server.sanitizer import LEAK_MARKERS, guarded_stops
    assert guarded_stops(["END", ""], enabled=False) == ["END"]
    got = guarded_stops(["END", "<|im_end|>"])
    assert got[:2] == ["END", "<|im_end|>"] and got.count("<|im_end|>") == 1
    assert set(LEAK_MARKERS) <= set(got)


def test_tool_call_dedupe():
    from atlas_b200.server.tool_parsers import ToolCall, dedupe_calls
    calls = [ToolCall("ls", '{"path": "/", "all": true}'), ToolCall("ls", '{"all":true,"path":"/"}'),
             ToolCall("ls", '{"path": "/tmp"}'), ToolCall("cat", '{"path": "/"}'), ToolCall("cat", "not json"),
             ToolCall("cat", "not json")]
    out = dedupe_calls(calls)
    assert [(c.name, c.arguments) for c in out] == [("ls", '{"path": "/", "all": true}'), ("ls", '{"path": "/tmp"}'),
                                                    ("cat", '{"path": "/"}'), ("cat", "not json")]
    assert out[0] is calls[0]


# ----------------------------------------------------------------------------------------------------- kernel scratch
@pytest.mark.parametrize("preset,tp", [("qwen3-30b-a3b", 1), ("llama3-70b", 1), ("llama3-70b", 8)])
def test_attention_scratch_is_reserved_once_and_never_replaced(preset, tp, monkeypatch):
    """The split-K decode attention partials live in a persistent buffer whose address CUDA graphs capture.  Sized for
    the worst padded batch up front, the buffer must be the same object for every batch size, and once a graph
    exists a larger request must raise instead of reallocating."""
    from atlas_b200.config import PRESETS
    from atlas_b200.ops import cuda as K
    from atlas_b200.runner import _GRAPH_BATCH_SIZES
    cfg = PRESETS[preset]()
    hq, hkv, d = cfg.num_attention_heads // tp, max(1, cfg.num_key_value_heads // tp), cfg.head_dim
    monkeypatch.setattr(K, "_scratch_alloc", lambda n, dev: torch.zeros(n, dtype=torch.uint8))
    monkeypatch.setattr(K, "_scratch", {})
    monkeypatch.setattr(K, "_scratch_frozen", False)
    dev = torch.device("cpu")
    sizes = [b for b in _GRAPH_BATCH_SIZES if b <= 128]
    po, pml = K.attention_scratch_bytes(sizes, hq, hkv, d, 8192, 148)
    assert po > 0
    K.reserve_scratch("attn_part_o", po, dev)
    K.freeze_scratch()
    base = K.scratch("attn_part_o", 1, dev).data_ptr()
    for b in sizes:
        s = K.decode_splits(b, hkv, 8192, 148)
        if s > 1:
            assert K.scratch("attn_part_o", b * hq * s * d * 4, dev).data_ptr() == base
    with pytest.raises(K.KernelError):
        K.scratch("attn_part_o", max(po, 1 << 20) + 1, dev)


def test_router_variants_reference():
    """Selection bias, group-limited routing, sqrt-softplus scores, static hash selection and the weight scale, each
    against a direct restatement of the published routing rule."""
    import torch
    from atlas_b200.ops import reference as ref
    torch.manual_seed(0)
    lg = torch.randn(7, 64)
    w, i = ref.moe_route(lg, 4, True)
    w0 = torch.softmax(lg, -1).topk(4).values
    assert torch.allclose(w, w0 / w0.sum(-1, keepdim=True))
    b = torch.randn(64) * 0.1
    w, i = ref.moe_route(lg, 4, True, "sigmoid", b, 8, 3, 2.5)
    sc = torch.sigmoid(lg)
    s2 = sc + b
    gi = s2.view(7, 8, 8).topk(2, -1).values.sum(-1).topk(3, -1).indices
    mask = torch.zeros(7, 8).scatter_(1, gi, 1)[..., None].expand(7, 8, 8).reshape(7, 64).bool()
    ti = s2.masked_fill(~mask, 0.0).topk(4, -1).indices
    tw = sc.gather(1, ti)
    assert (ti == i).all() and torch.allclose(tw / (tw.sum(-1, keepdim=True) + 1e-20) * 2.5, w, atol=1e-6)
    tab = torch.randint(0, 64, (100, 4), dtype=torch.int32)
    tok = torch.randint(0, 100, (7,), dtype=torch.int32)
    w, i = ref.moe_route(lg, 4, True, "sqrtsoftplus", None, 0, 0, 1.5, tab, tok)
    assert (i == tab[tok.long()]).all() and torch.allclose(w.sum(-1), torch.full((7,), 1.5))
    sp = torch.sqrt(torch.nn.functional.softplus(lg)).gather(1, i.long())
    assert torch.allclose(w, sp / sp.sum(-1, keepdim=True) * 1.5, atol=1e-6)


def test_memory_watchdog_levels_and_engine_hooks():
    """Soft floor pauses admission (with hysteresis), hard floor trips the latch once; driven by fake samples."""
    from atlas_b200.utils.watchdog import Level, MemorySample, MemoryWatchdog, WatchdogConfig, decide, preflight
    cfg = WatchdogConfig(soft_device_free=1000, hard_device_free=100, soft_host_available=0, hard_host_available=0,
                         recover_factor=2.0)
    mk = lambda free: MemorySample(free, 10000, 0)
    assert decide(mk(5000), cfg) == Level.OK and decide(mk(999), cfg) == Level.SOFT and decide(mk(99), cfg) == Level.HARD
    assert decide(mk(1500), cfg, Level.SOFT) == Level.SOFT and decide(mk(2001), cfg, Level.SOFT) == Level.OK
    feed = iter([5000, 900, 1500, 2500, 50, 50])
    events = []
    wd = MemoryWatchdog(cfg, lambda: mk(next(feed)), on_soft=lambda on: events.append(("soft", on)),
                        on_hard=lambda why: events.append(("hard", why)))
    levels = [wd.poll() for _ in range(6)]
    assert levels == [Level.OK, Level.SOFT, Level.SOFT, Level.OK, Level.HARD, Level.HARD]
    assert events[0] == ("soft", True) and events[1] == ("soft", False) and events[2][0] == "hard" and len(events) == 3
    assert "out of memory" in events[2][1]
    assert preflight(8 << 30, 4 << 30, 16 << 30) is None and "needs" in preflight(8 << 30, 8 << 30, 16 << 30)
    # paused admission: a waiting request is not admitted, running work continues
    import torch
    from atlas_b200.config import EngineConfig, tiny_dense
    from atlas_b200.engine import LLMEngine
    from atlas_b200.models import build_model
    from atlas_b200.sampling import SamplingParams
    eng = LLMEngine(build_model(tiny_dense("float32"), device="cpu").init_random(0), EngineConfig(num_kv_blocks=32, max_seq_len=64))
    eng.scheduler.admission_paused = True
    eng.add_request([1, 2, 3], SamplingParams(max_tokens=2, ignore_eos=True))
    assert eng.step() == [] and len(eng.scheduler.waiting) == 1
    eng.scheduler.admission_paused = False
    while eng.has_unfinished():
        eng.step()
    assert not eng.scheduler.waiting


def test_red_zone_guards_and_block_poison():
    import torch
    from atlas_b200.utils.guards import CANARY, GuardedAllocator, poison_block, zero_block
    ga = GuardedAllocator(zone_bytes=64)
    a = ga.alloc("a", (3, 5), torch.float32, "cpu")
    b = ga.alloc("b", (7,), torch.bfloat16, "cpu")
    assert a.shape == (3, 5) and float(a.abs().sum()) == 0 and ga.scan() == []
    a.fill_(1.0)
    b.fill_(2.0)
    assert ga.scan() == []                                # writes inside the payload leave the bands alone
    raw = ga.entries[0].raw
    raw[64 + 60 + 3] = 7                                   # one byte past the end of `a` (60 payload bytes)
    bad = ga.scan()
    assert len(bad) == 1 and bad[0].name == "a" and bad[0].side == "above" and bad[0].offset == 3 and bad[0].value == 7
    ga.repair()
    assert ga.scan() == [] and int(raw[0]) == CANARY
    assert [e["name"] for e in ga.ledger()] == ["a", "b"] and ga.ledger()[0]["bytes"] == 60
    k = torch.zeros(4, 16, 2, 8, dtype=torch.float8_e4m3fn)
    v = torch.zeros(4, 16, 2, 8, dtype=torch.bfloat16)
    poison_block((k, v), 2)
    assert float(k[2].float().min()) == 448.0 and float(v[2].float().min()) > 1e30 and float(k[1].float().abs().sum()) == 0
    zero_block((k, v), 2)
    assert float(k.float().abs().sum()) == 0 and float(v.float().abs().sum()) == 0


def test_spec_gate_uses_the_agreed_measurement():
    """Two ranks time the same probe differently; with the agreement hook (here: the maximum of both) they reach the same
    verdict, without it they would not."""
    from atlas_b200.sched.spec import MtpGate

    def run(times_spec, times_plain, agree):
        g = MtpGate(enabled=True, probe_steps=4, agree=agree)
        for t in times_spec:
            g.record(True, t, 8)
        for t in times_plain:
            g.record(False, t, 4)
        return g.mode

    a = ([0.010] * 4, [0.0049] * 4)          # rank 0: spec 800 tok/s vs plain 816 tok/s -> plain
    b = ([0.010] * 4, [0.0052] * 4)          # rank 1: spec 800 vs plain 769 -> spec
    assert run(*a, None) == "plain" and run(*b, None) == "spec"
    shared = {"spec": None, "plain": None}

    def make(rank_vals_other):
        it = iter(rank_vals_other)
        return lambda v: [max(x, y) for x, y in zip(v, next(it))]
    other_of_a = [[0.040, 32.0], [0.0208, 16.0]]     # what rank 1 measured for the two probes
    other_of_b = [[0.040, 32.0], [0.0196, 16.0]]     # what rank 0 measured
    assert run(*a, make(other_of_a)) == run(*b, make(other_of_b)) == "spec"


def test_batched_record_io_through_io_uring(tmp_path):
    """The file tier's batched path: records written from and read into host rows through one io_uring submission must
    be what positional reads / writes of the same offsets see; more records than the queue depth, a ragged last batch,
    and a read past the end of the file reports an error instead of returning short data."""
    import os

    from atlas_b200 import runtime_native as rn
    from atlas_b200.kv.host_tier import DiskKVTier
    if not rn.uring_available():
        pytest.skip("io_uring is not available to this process")
    rec_bytes, n = 4096 + 512, 150
    tier = DiskKVTier(rec_bytes, 200, str(tmp_path))
    try:
        assert tier._uring()
        g = torch.Generator().manual_seed(1)
        rows = torch.randint(0, 256, (n, rec_bytes), generator=g, dtype=torch.uint8)
        recs = torch.randperm(200, generator=g)[:n].tolist()
        tier.write_many(recs, [rows[i] for i in range(n)])
        for i in (0, 7, n - 1):                                       # what a plain positional read sees
            assert os.pread(tier.fd, rec_bytes, recs[i] * rec_bytes) == rows[i].numpy().tobytes()
        back = torch.zeros_like(rows)
        tier.read_many(recs, [back[i] for i in range(n)])
        assert torch.equal(back, rows) and tier.records_out == n and tier.records_in == n
        # the plain path moves the same bytes
        tier._uring_ok = False
        back2 = torch.zeros_like(rows)
        tier.read_many(recs[:5], [back2[i] for i in range(5)])
        assert torch.equal(back2[:5], rows[:5])
        buf = torch.zeros(rec_bytes, dtype=torch.uint8)
        with pytest.raises(OSError):
            rn.uring_rw(tier.fd, False, [200 * rec_bytes], [buf.data_ptr()], rec_bytes)
    finally:
        tier.close()
