"""Multi-process control plane on CPU: a leader engine and follower engines (threads over the in-process fake
communicator, TP=2 sharded weights) must stay in lock-step — same plans, same tokens as a single-process engine —
including leader-only decisions (stop checkers, timeouts, aborts), and a follower must give up with an error, not
hang, when the leader disappears."""
import threading
import time

import pytest
import torch

from atlas_b200.config import EngineConfig, tiny_dense, tiny_hybrid
from atlas_b200.engine import LLMEngine
from atlas_b200.layers import ParallelCtx
from atlas_b200.models import build_model
from atlas_b200.parallel.comm import CommError, FakeWorld
from atlas_b200.parallel.worker import DistributedEngine, StepControl, worker_loop
from atlas_b200.sampling import SamplingParams
from atlas_b200.utils import fault


def _prompts(n=4, length=24, seed=2):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def _ecfg(**kw):
    return EngineConfig(block_size=16, num_kv_blocks=64, max_num_seqs=8, max_prefill_tokens=48, **kw)


def _run_world(mk, ecfg, leader_fn, world_size=2):
    """Build one engine per fake rank (TP-sharded), run ``leader_fn(dist_engine)`` on rank 0 and the worker loop on
    the others.  Returns (leader result, follower engines)."""
    data = FakeWorld(world_size, timeout_s=20.0)      # tensor collectives
    ctrl = FakeWorld(world_size, timeout_s=20.0)      # control plane
    followers = [None] * world_size

    def rank_fn(r):
        comm = data.comm(r)
        pctx = ParallelCtx(tp_rank=r, tp_size=world_size, ep_rank=r, ep_size=world_size, comm=comm, ep_comm=comm)
        model = build_model(mk(), pctx).init_random(0)
        eng = LLMEngine(model, ecfg)
        control = StepControl(ctrl.comm(r), heartbeat_s=0.05)
        if r == 0:
            de = DistributedEngine(eng, control)
            try:
                return leader_fn(de)
            finally:
                de.shutdown()
        followers[r] = eng
        return worker_loop(eng, control)

    outs = data.run(rank_fn, timeout_s=120.0)
    return outs[0], followers


def _drain(de, want_ids):
    done = {}
    while len(done) < len(want_ids):
        for o in de.step():
            if o.finished:
                done[o.request_id] = o
    return done


@pytest.mark.parametrize("mk", [tiny_dense, tiny_hybrid])
def test_leader_and_followers_match_single_process(mk):
    prompts = _prompts()
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    base = LLMEngine(build_model(mk()).init_random(0), _ecfg()).generate(prompts, sp)

    def leader(de):
        ids = [de.add_request(p, SamplingParams(max_tokens=10, ignore_eos=True)) for p in prompts[:2]]
        de.step()                      # requests arriving while others are in flight
        ids += [de.add_request(p, SamplingParams(max_tokens=10, ignore_eos=True)) for p in prompts[2:]]
        done = _drain(de, ids)
        return [done[i].output_tokens for i in ids]

    toks, followers = _run_world(mk, _ecfg(), leader)
    assert toks == [o.output_tokens for o in base]
    for f in followers[1:]:
        assert not f.has_unfinished()
        assert f.stats.generation_tokens == 40
        f.pool.check_invariants()


def test_leader_only_decisions_are_replayed():
    """A stop checker (host-side, leader only), an abort and a timeout all reach the followers as outcomes / events."""
    prompts = _prompts(3)

    def leader(de):
        a = de.add_request(prompts[0], SamplingParams(max_tokens=32, ignore_eos=True),
                           stop_checker=lambda seq: seq.num_output_tokens >= 3)
        b = de.add_request(prompts[1], SamplingParams(max_tokens=32, ignore_eos=True))
        c = de.add_request(prompts[2], SamplingParams(max_tokens=10_000, ignore_eos=True), timeout_s=0.15)
        seen = {}
        steps = 0
        while len(seen) < 3:
            for o in de.step():
                if o.finished:
                    seen[o.request_id] = o
            steps += 1
            if steps == 4:
                assert de.abort(b)
                seen[b] = None
            time.sleep(0.02)
        return seen[a].finish_reason, len(seen[a].output_tokens), seen[c].finish_reason, de.pool.num_free

    (fin_a, n_a, fin_c, leader_free), followers = _run_world(tiny_dense, _ecfg(max_seq_len=512), leader)
    assert (fin_a, n_a, fin_c) == ("stop", 3, "timeout")
    for f in followers[1:]:
        assert not f.has_unfinished()
        f.pool.check_invariants()
        assert f.pool.num_free == leader_free        # same blocks in use (only prefix-cache entries remain)


def test_speculative_followers_stay_in_step():
    prompts = _prompts()
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    base = LLMEngine(build_model(tiny_hybrid()).init_random(0), _ecfg()).generate(prompts, sp)
    cfg = _ecfg(speculative=True, num_drafts=2, mtp_gate=True)

    def leader(de):
        ids = [de.add_request(p, SamplingParams(max_tokens=10, ignore_eos=True)) for p in prompts]
        done = _drain(de, ids)
        return [done[i].output_tokens for i in ids], de.stats.spec_proposed

    (toks, proposed), followers = _run_world(tiny_hybrid, cfg, leader)
    assert toks == [o.output_tokens for o in base]
    assert proposed > 0


def test_follower_gives_up_when_leader_vanishes():
    """Host-side failure injection: the leader never sends another plan; the follower's bounded wait raises, poisons
    its communicator and trips the fault latch instead of hanging."""
    fault.FAULT_LATCH.reset_for_tests()
    ctrl = FakeWorld(2, timeout_s=0.3)
    eng = LLMEngine(build_model(tiny_dense()).init_random(0), _ecfg())
    control = StepControl(ctrl.comm(1))
    err = []

    def body():
        try:
            worker_loop(eng, control)
        except CommError as e:
            err.append(e)

    t = threading.Thread(target=body, daemon=True)
    t0 = time.monotonic()
    t.start()
    t.join(5.0)
    assert not t.is_alive() and time.monotonic() - t0 < 3.0
    assert err and "timed out" in str(err[0])
    assert control.comm.unhealthy and fault.FAULT_LATCH.tripped
    fault.FAULT_LATCH.reset_for_tests()


def test_vocab_parallel_greedy_and_leader_only_processors_agree_on_the_logits_path():
    """Plain greedy steps exchange (max, index) pairs instead of gathering logits; a request whose leader-side sampling
    needs the whole row (a logits processor that only exists on rank 0) must switch every rank to the gather."""
    prompts = _prompts()
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    base = LLMEngine(build_model(tiny_dense()).init_random(0), _ecfg()).generate(prompts[:2], sp)
    seen = []

    def ban_token(row, seq):
        seen.append(int(row.shape[-1]))
        return row

    def leader(de):
        assert de.engine.model.vocab_parallel
        a = de.add_request(prompts[0], SamplingParams(max_tokens=8, ignore_eos=True))
        for _ in range(3):
            de.step()                                   # greedy-only steps: pair exchange
        b = de.add_request(prompts[1], SamplingParams(max_tokens=8, ignore_eos=True), logits_processors=[ban_token])
        done = _drain(de, [a, b])
        return [done[a].output_tokens, done[b].output_tokens]

    got, followers = _run_world(tiny_dense, _ecfg(), leader)
    assert got == [o.output_tokens for o in base]
    assert seen and all(v == tiny_dense().vocab_size for v in seen)      # the processor saw full-vocabulary rows
