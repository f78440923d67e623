"""Sequence-parallel tensor parallelism on one GPU: the ranks of a group run one after another over separate buffers.

The three kernels of a layer half only depend forwards (GEMM with the reduce-scatter epilogue -> owner-side reduce +
norm + quantise + gather -> GEMM over the gathered rows), so executing phase by phase, every rank in turn, satisfies
every flag before anything waits on it.  Checked against a plain fp32 computation of the same layer half."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt().clamp_min(1e-12))


@pytest.mark.parametrize("T,world,H,Kr,plus_one", [(1000, 4, 1024, 512, False), (300, 8, 512, 256, True), (2048, 2, 2048, 1024, False),
                                                   # decode-size steps: the rows of the single 128-row block are owned rank by rank
                                                   (128, 8, 512, 256, False), (100, 4, 1024, 512, True), (5, 8, 512, 256, False),
                                                   (64, 2, 1024, 512, False)])
def test_gemm_reduce_scatter_norm_gather_gemm(T, world, H, Kr, plus_one):
    from atlas_b200 import quant as Q
    from atlas_b200.ops import Act, LinearWeight, linear
    from atlas_b200.ops import cuda as K
    from atlas_b200.parallel.seqpar import SeqParallelArea
    K.load()
    torch.manual_seed(3)
    eps = 1e-6
    xs = [(torch.randn(T, Kr, device=DEV) * 0.5).bfloat16() for _ in range(world)]
    ws = [LinearWeight.from_dense(torch.randn(H, Kr, device=DEV) * 0.05, "fp8_block") for _ in range(world)]
    resid = torch.randn(T, H, device=DEV).bfloat16()
    norm_w = (torch.randn(H, device=DEV) * 0.2 + (0.0 if plus_one else 1.0)).bfloat16()
    w2 = LinearWeight.from_dense(torch.randn(384, H, device=DEV) * 0.05, "fp8_block")
    areas = [SeqParallelArea(r, world, T, H, DEV, wait_cycles=50_000_000) for r in range(world)]
    bases = [a.allocate_local() for a in areas]
    for a in areas:
        a.connect(bases)
    # fp32 statement of the same computation
    acts = [Act(x=x) for x in xs]
    want_sum = sum(Q.fp8_block_gemm_ref(*a.fp8(), w.weight, w.scale, out_dtype=torch.float32) for a, w in zip(acts, ws))
    h = want_sum + resid.float()
    weff = norm_w.float() + (1.0 if plus_one else 0.0)
    normed = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * weff
    want_y = normed @ w2.dequantized().float().t()

    for r, a in enumerate(areas):                                   # phase 1: partial tiles to the row owners
        a.gemm_rs(acts[r], ws[r])
    shards = [a.residual_shard(resid) for a in areas]
    gathered = [a.reduce_norm(shards[r], norm_w, eps, plus_one) for r, a in enumerate(areas)]    # phase 2
    ys = [linear(g, w2) for g in gathered]                          # phase 3: GEMM over the gathered rows
    torch.cuda.synchronize()
    assert K.check_status() == 0
    got_h = torch.cat(shards)
    assert got_h.shape == (T, H)
    assert _rel(got_h, h) < 1e-2
    for g in gathered[1:]:                                          # every rank holds the same gathered rows
        assert torch.equal(g.q.view(torch.uint8), gathered[0].q.view(torch.uint8)) and torch.equal(g.s, gathered[0].s)
    deq = gathered[0].q.float().view(T, -1, 128) * gathered[0].s.contiguous()[..., None]
    assert _rel(deq.view(T, H), normed) < 4e-2
    for y in ys:
        assert torch.equal(y, ys[0])
        assert _rel(y, want_y) < 4e-2
    # second layer half on the same areas: the flags carry epochs, nothing is reset; bf16 hidden gather at the end
    for r, a in enumerate(areas):
        a.gemm_rs(acts[(r + 1) % world], ws[(r + 1) % world])
    for r, a in enumerate(areas):
        a.reduce_hidden_start(shards[r])
    hid = [a.hidden_wait() for a in areas]
    torch.cuda.synchronize()
    assert K.check_status() == 0
    want_h2 = got_h.float() + want_sum
    for x in hid:
        assert torch.equal(x, hid[0]) and x.shape == (T, H)
    assert _rel(hid[0], want_h2) < 1e-2
    assert torch.equal(torch.cat(shards), hid[0])


def test_gathered_gemm_wait_expires_cleanly():
    """Rows that never arrive: the producer's bounded wait gives up, the kernel returns, the status word names the
    site, and the next ordinary launch on the same context works."""
    from atlas_b200.ops import Act, LinearWeight, linear
    from atlas_b200.ops import cuda as K
    K.load()
    torch.manual_seed(0)
    T, H = 256, 512
    x = torch.randn(T, H, device=DEV).bfloat16()
    w = LinearWeight.from_dense(torch.randn(256, H, device=DEV) * 0.05, "fp8_block")
    q, s = K.quant_fp8(x)
    flags = torch.zeros(T // 8, dtype=torch.int32, device=DEV)        # nothing ever raises these
    epoch = torch.ones(4, dtype=torch.int32, device=DEV)
    act = Act(q=q, s=s, dtype=torch.bfloat16, ready=(flags.data_ptr(), epoch.data_ptr(), 2_000_000))
    linear(act, w)
    torch.cuda.synchronize()
    st = K.check_status()
    assert st & 0xFF == 2 and (st >> 8) & 0xFFFFFF == 0x620, hex(st)   # kFlagTimeout at the gathered-rows wait
    flags.fill_(1)
    y = linear(act, w)
    want = linear(Act(q=q, s=s, dtype=torch.bfloat16), w)
    torch.cuda.synchronize()
    assert K.check_status() == 0 and torch.equal(y, want)


def test_allreduce_wait_expires_and_poisons_then_recovers():
    """`atlas_allreduce_bf16` with world = 2 on ONE GPU: the second "rank" is a local buffer whose flags nobody raises,
    so the kernel's bounded wait on the peer runs out.  The kernel must return, the status word must name the
    barrier site, a communicator reading it must poison itself, and after the word is cleared a healthy call works."""
    import ctypes as C
    from atlas_b200.ops import cuda as K
    from atlas_b200.parallel.comm import CommBackend, CommError
    K.load()
    lib = K.lib()
    vp, i, ll, sz = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t
    lib.atlas_allreduce_bf16.argtypes = [i, C.POINTER(vp), C.POINTER(vp), i, i, vp, vp, sz, sz, vp, i, vp, ll, vp]
    slot = 1 << 20
    data = [torch.zeros(2 * slot, dtype=torch.uint8, device=DEV) for _ in range(2)]
    flags = [torch.zeros(2 * 256 * 8, dtype=torch.int32, device=DEV) for _ in range(2)]
    state = torch.zeros(4, dtype=torch.int32, device=DEV)
    x = torch.randn(4096, device=DEV).bfloat16()
    y = torch.empty_like(x)
    d = K._dev(x)
    darr = (vp * 8)(*([t.data_ptr() for t in data] + [None] * 6))
    farr = (vp * 8)(*([t.data_ptr() for t in flags] + [None] * 6))
    for kind in (0, 1):
        rc = lib.atlas_allreduce_bf16(kind, darr, farr, 0, 2, x.data_ptr(), y.data_ptr(), x.numel() * 2, slot, state.data_ptr(), 2,
                                      K._status_ptr[d], 1_000_000, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()                       # the kernel came back by itself
        st = K.check_status(clear=False)
        assert st & 0xFF == 2 and ((st >> 8) & 0xFFFFFF) in (0x500, 0x501), hex(st)

        class _Probe(CommBackend):
            name = "probe"

            def check(self):
                s = K.check_status()
                if s:
                    self.poison(f"peer wait expired ({s:#x})")
                    raise CommError("expired")
        c = _Probe()
        with pytest.raises(CommError):
            c.check()
        assert c.unhealthy
        with pytest.raises(CommError):
            c._guard()
        assert K.check_status() == 0                   # cleared by the read above
    # world = 1 degenerates to a copy through the slot and must be healthy after the expired calls
    state.zero_()
    rc = lib.atlas_allreduce_bf16(0, darr, farr, 0, 1, x.data_ptr(), y.data_ptr(), x.numel() * 2, slot, state.data_ptr(), 2,
                                  K._status_ptr[d], 1_000_000, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and K.check_status() == 0 and torch.equal(x, y)
