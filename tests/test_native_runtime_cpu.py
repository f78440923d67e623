"""Native host runtime (C++): block pool and radix tree against their Python twins on random operation streams,
fault latch, direct-I/O reader, and the engine running on the native pool."""
import os
import random

import pytest
import torch

from atlas_b200 import runtime_native as N
from atlas_b200.kv import BlockPool, RadixCache
from atlas_b200.kv.block_manager import OutOfBlocks


def test_pool_matches_python_twin():
    rnd = random.Random(1)
    a, b = BlockPool(32, 16), N.NativeBlockPool(32, 16)
    held = []
    for _ in range(2000):
        op = rnd.random()
        if op < 0.4:
            n = rnd.randrange(1, 6)
            try:
                x = a.alloc(n)
            except OutOfBlocks:
                with pytest.raises(OutOfBlocks):
                    b.alloc(n)
                continue
            assert b.alloc(n) == x
            held.append(x)
        elif op < 0.6 and held:
            x = rnd.choice(held)
            a.inc_ref(x)
            b.inc_ref(x)
            held.append(list(x))
        elif held:
            x = held.pop(rnd.randrange(len(held)))
            assert a.free(x) == b.free(x)
        assert a.num_free == b.num_free
    b.check_invariants()
    assert [a.ref_count(i) for i in range(32)] == [b.ref_count(i) for i in range(32)]
    for x in held:
        a.free(x), b.free(x)
    with pytest.raises(ValueError):
        b.free([0])
    with pytest.raises(ValueError):
        b.inc_ref([0])


def test_radix_matches_python_twin():
    rnd = random.Random(2)
    pa, pb = BlockPool(64, 2), N.NativeBlockPool(64, 2)
    ra, rb = RadixCache(pa), N.NativeRadix(pb)
    for _ in range(400):
        toks = [rnd.randrange(3) for _ in range(rnd.randrange(2, 14))]
        op = rnd.random()
        if op < 0.5:
            n = pa.blocks_for_tokens(len(toks))
            if pa.num_free < n:
                assert ra.evict(n) == rb.evict(n)
            if pa.num_free < n:
                continue
            xa, xb = pa.alloc(n), pb.alloc(n)
            assert xa == xb
            ra.insert(toks, xa)
            rb.insert(toks, xb)
            pa.free(xa), pb.free(xb)
        elif op < 0.9:
            m = ra.match(toks)
            blocks, nodes = rb.match(toks)
            assert m.blocks == blocks
            ra.release(m.nodes), pa.free(m.blocks)
            rb.release(nodes), pb.free(blocks)
        else:
            k = rnd.randrange(1, 5)
            assert ra.evict(k) == rb.evict(k)
        assert pa.num_free == pb.num_free and ra.num_nodes == rb.num_nodes
    assert ra.evictable_blocks() == rb.evictable_blocks()
    pb.check_invariants()


def test_fault_latch_is_one_shot():
    N.lib().atlas_fault_reset_for_tests()
    assert not N.fault_tripped() and N.fault_reason() is None
    assert N.fault_trip("first") and not N.fault_trip("second")
    assert N.fault_tripped() and N.fault_reason() == "first"
    N.lib().atlas_fault_reset_for_tests()


def test_direct_io_reader(tmp_path):
    data = os.urandom(3 * (1 << 20) + 12345)
    p = tmp_path / "blob.bin"
    p.write_bytes(data)
    for off, ln, chunk in [(0, len(data), 1 << 20), (4097, 2_000_003, 256 << 10), (len(data) - 100, 100, 1 << 20)]:
        buf = torch.empty(ln, dtype=torch.uint8)
        got = N.read_file_into(str(p), off, ln, buf.data_ptr(), threads=4, chunk=chunk)
        assert got == ln and bytes(buf.numpy().tobytes()) == data[off:off + ln]
    buf = torch.empty(1000, dtype=torch.uint8)
    assert N.read_file_into(str(p), len(data) - 10, 1000, buf.data_ptr()) == 10        # short read at end of file
    with pytest.raises(OSError):
        N.read_file_into(str(tmp_path / "missing"), 0, 10, buf.data_ptr())


def test_engine_on_native_pool(monkeypatch):
    from atlas_b200.config import EngineConfig, tiny_dense
    from atlas_b200.engine import LLMEngine
    from atlas_b200.models import build_model
    from atlas_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (40,), generator=g).tolist() for _ in range(4)]
    sp = SamplingParams(max_tokens=24, ignore_eos=True)
    model = build_model(tiny_dense()).init_random(0)
    want = [o.output_tokens for o in LLMEngine(model, EngineConfig(num_kv_blocks=14, max_num_seqs=8)).generate(prompts, sp)]
    monkeypatch.setenv("ATLAS_NATIVE_RUNTIME", "1")
    eng = LLMEngine(model, EngineConfig(num_kv_blocks=14, max_num_seqs=8))
    assert isinstance(eng.pool, N.NativeBlockPool)
    assert [o.output_tokens for o in eng.generate(prompts, sp)] == want
    eng.pool.check_invariants()
