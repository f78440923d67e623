"""Two-level residency (LRU / ARC, pins, capped cold tier) and the D-Cut verify-depth planner."""
import math
import random

import pytest

from atlas_b200.kv.residency import FileSwapStore, MemSwapStore, Residency
from atlas_b200.sched import dcut


@pytest.mark.parametrize("policy", ["lru", "arc"])
def test_residency_spill_promote_and_never_reject(policy, tmp_path):
    cold = FileSwapStore(str(tmp_path / "swap.bin"), 16) if policy == "lru" else MemSwapStore(16)
    r = Residency(4, 16, cold, policy)
    for k in range(10):
        r.put(k, bytes([k]) * 16)
    assert len(r.hot_keys) == 4 and len(r.cold_keys) == 6 and r.stats["spills"] == 6
    for k in range(10):                                   # every key is still readable; cold ones are promoted
        assert r.get(k) == bytes([k]) * 16
    assert r.stats["cold_hits"] >= 6 and r.get(99) is None and r.stats["misses"] == 1
    r.remove(3)
    assert 3 not in r and r.get(3) is None


def test_residency_pins_and_capped_cold_tier():
    r = Residency(2, 8, MemSwapStore(8, capacity=2), "lru")
    r.put("a", b"A" * 8)
    r.put("b", b"B" * 8)
    assert r.get("a", pin=True) == b"A" * 8               # "a" is held by a reader
    r.put("c", b"C" * 8)                                  # must spill "b", not the pinned "a"
    assert "a" in r.hot_keys and "b" in r.cold_keys
    for k in "defg":
        r.put(k, k.encode() * 8)
    assert "a" in r.hot_keys                              # still pinned
    assert len(r.cold_keys) <= 2 and r.stats["drops"] >= 1   # the capped cold tier dropped its coldest keys
    r.unpin("a")
    r.put("h", b"h" * 8)
    r.put("i", b"i" * 8)
    assert "a" not in r.hot_keys


def test_arc_keeps_the_frequent_set_through_a_scan():
    def run(policy):
        r = Residency(8, 4, MemSwapStore(4), policy)
        hot = list(range(4))
        for _ in range(3):
            for k in hot:
                r.put(k, b"x" * 4) if k not in r else r.get(k)
        for k in range(100, 140):                         # one-time scan, larger than the hot tier
            r.put(k, b"y" * 4)
            for h in hot[:2]:
                r.get(h)
        return sum(1 for k in hot[:2] if k in r.hot_keys)
    assert run("arc") == 2


def test_dcut_keeps_prefixes_and_ranks_across_the_batch():
    ln = math.log
    lp = [[ln(.99), ln(.98), ln(.97)], [ln(.9), ln(.2), ln(.9)], [ln(.5), ln(.5), ln(.5)]]
    assert dcut.plan(lp, ratio=1.0) == [3, 3, 3]
    half = dcut.plan(lp, ratio=0.5)                       # 6 prunable positions, 3 kept: the confident sequence keeps depth
    assert half == [3, 1, 2] and all(c >= 1 for c in half)
    assert dcut.plan(lp, ratio=0.25) == [2, 1, 1]
    assert dcut.snap_ratio(0.6) == 0.5 and dcut.snap_ratio(0.9) == 1.0
    wide = [[ln(.5)] * 3 for _ in range(12)]
    assert dcut.plan(wide, ratio=0.25, max_seqs=8) == [3] * 12            # beyond the width cap nothing is pruned
    assert sum(c + 1 for c in dcut.plan(wide, ratio=1.0, row_budget=30, max_seqs=16)) <= 30


def test_dcut_cost_model_and_estimator():
    ln = math.log
    lp = [[ln(.95), ln(.95), ln(.95), ln(.95)], [ln(.6), ln(.3), ln(.3), ln(.3)]]
    cheap = dcut.plan_cost_optimal(lp, None, base_cost=10.0, row_cost=0.01)
    dear = dcut.plan_cost_optimal(lp, None, base_cost=1.0, row_cost=2.0)
    assert cheap[0] == 4 and cheap[1] >= 2 and dear[1] == 1 and sum(dear) < sum(cheap)
    est = dcut.AcceptEstimator()
    rnd = random.Random(0)
    for _ in range(400):                                  # the verifier accepts far less than the drafter claims
        est.record(ln(.9), rnd.random() < 0.3)
    assert 0.2 < est.p_accept(ln(.9)) < 0.4
    assert dcut.plan_cost_optimal([[ln(.9)] * 4], est, base_cost=1.0, row_cost=0.5)[0] < \
        dcut.plan_cost_optimal([[ln(.9)] * 4], None, base_cost=1.0, row_cost=0.5)[0]
