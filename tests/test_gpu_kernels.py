"""sm_100a kernels vs the plain-PyTorch fp32 restatement of the same op (needs a B200)."""
import math

import pytest
import torch

from atlas_b200 import quant as Q
from atlas_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def K():
    from atlas_b200.ops import cuda as k
    k.load()
    return k


def _status_ok(K):
    torch.cuda.synchronize()
    st = K.check_status()
    assert st == 0, f"device status word {st:#x}"


def _rel_rms(a, b):
    a, b = a.float(), b.float()
    return float((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt().clamp_min(1e-12))


# ----------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (128, 256, 512), (1, 512, 256), (37, 384, 1024), (300, 640, 320),
                                    (1024, 4096, 4096)])
def test_gemm_bf16(K, M, N, K_):
    torch.manual_seed(0)
    a = (torch.randn(M, K_, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(N, K_, device=DEV) * 0.5).bfloat16()
    out = K.gemm_bf16(a, b)
    want = a.float() @ b.float().t()
    _status_ok(K)
    assert _rel_rms(out, want) < 6e-3
    torch.testing.assert_close(out.float(), want, atol=0.25, rtol=3e-2)


@pytest.mark.parametrize("M,N,K_", [(128, 128, 128), (5, 256, 512), (128, 1024, 4096), (200, 768, 1024), (1024, 6144, 4096),
                                    (64, 4096, 14336)])
def test_gemm_fp8_block(K, M, N, K_):
    torch.manual_seed(1)
    x = (torch.randn(M, K_, device=DEV)).bfloat16()
    w = torch.randn(N, K_, device=DEV) * 0.05
    wq, ws = Q.quantize_fp8_block(w)
    xq, xs = K.quant_fp8(x)
    xq_ref, xs_ref = Q.per_token_group_quant_fp8(x)
    # scales agree to an ulp (PyTorch divides by a scalar as a reciprocal multiply on CUDA), so a few codes
    # that sit on a rounding boundary may differ by one step: compare codes statistically, values closely
    torch.testing.assert_close(xs.contiguous(), xs_ref, rtol=1e-6, atol=0)
    mismatch = (xq.view(torch.uint8) != xq_ref.view(torch.uint8)).float().mean().item()
    assert mismatch < 0.02, mismatch
    deq = xq.float().view(M, -1, 128) * xs.contiguous()[..., None]
    assert _rel_rms(deq.view(M, K_), x) < 4e-2
    out = K.gemm_fp8_block(xq, xs, wq, ws)
    want = Q.fp8_block_gemm_ref(xq, xs.contiguous(), wq, ws, out_dtype=torch.float32)
    _status_ok(K)
    assert _rel_rms(out, want) < 5e-3


@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (5, 512, 256), (300, 640, 1024), (130, 200, 448), (1024, 4096, 4096)])
def test_gemm_nvfp4_w4a16(K, M, N, K_):
    """Packed E2M1 weights + e4m3 block scales + fp32 global scale, widened inside the kernel, against the fp32 product
    with the dequantised weights (the widening itself is exact, so only bf16 activations / output rounding remain)."""
    torch.manual_seed(3)
    x = torch.randn(M, K_, device=DEV).bfloat16()
    w = torch.randn(N, K_, device=DEV) * 0.05
    packed, bs, gs = Q.quantize_nvfp4(w)
    out = K.gemm_nvfp4(x, packed, bs, gs)
    want = x.float() @ Q.dequantize_nvfp4(packed, bs, gs).t()
    _status_ok(K)
    assert _rel_rms(out, want) < 6e-3
    # one global scale per output row (fused projections quantised separately)
    gs_rows = (torch.rand(N, device=DEV) + 0.5) * gs.float().reshape(-1)[0]
    out2 = K.gemm_nvfp4(x, packed, bs, gs_rows)
    want2 = x.float() @ Q.dequantize_nvfp4(packed, bs, gs_rows).t()
    _status_ok(K)
    assert _rel_rms(out2, want2) < 6e-3


@pytest.mark.parametrize("bn,splits", [(64, 1), (64, 4), (128, 1), (128, 3), (256, 1), (256, 2)])
def test_gemm_tile_and_split_variants(K, monkeypatch, bn, splits):
    monkeypatch.setattr(K, "_FORCE_BLOCK_N", bn)
    monkeypatch.setattr(K, "_FORCE_SPLITS", splits)
    torch.manual_seed(2)
    M, N, K_ = 130, 520, 2048
    x = torch.randn(M, K_, device=DEV).bfloat16()
    w = torch.randn(N, K_, device=DEV) * 0.05
    wq, ws = Q.quantize_fp8_block(w)
    xq, xs = K.quant_fp8(x)
    out = K.gemm_fp8_block(xq, xs, wq, ws)
    want = Q.fp8_block_gemm_ref(xq, xs.contiguous(), wq, ws, out_dtype=torch.float32)
    assert _rel_rms(out, want) < 5e-3
    a = x
    b = (w * 10).bfloat16()
    out2 = K.gemm_bf16(a, b)
    assert _rel_rms(out2, a.float() @ b.float().t()) < 6e-3
    # same call twice gives identical bits (split reduction order is fixed)
    out3 = K.gemm_fp8_block(xq, xs, wq, ws)
    _status_ok(K)
    assert torch.equal(out, out3)


# ----------------------------------------------------------------------------- norm / activation
@pytest.mark.parametrize("T,H", [(1, 256), (7, 4096), (33, 2048), (5, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(K, T, H, with_res):
    torch.manual_seed(3)
    x = torch.randn(T, H, device=DEV).bfloat16()
    r = torch.randn(T, H, device=DEV).bfloat16() if with_res else None
    w = (torch.rand(H, device=DEV) + 0.5).bfloat16()
    y, ro = K.rmsnorm(x, w, 1e-6, r, False, quant=False)
    yr, rr = ref.rmsnorm(x, w, 1e-6, r, False)
    torch.testing.assert_close(y.float(), yr.float(), atol=2e-2, rtol=2e-2)
    if with_res:
        assert torch.equal(ro, rr)
    q, s, _ = K.rmsnorm(x, w, 1e-6, r, False, quant=True)
    qr, sr, _ = ref.rmsnorm_quant_fp8(x, w, 1e-6, r, False)
    deq = q.float().view(T, -1, 128) * s.contiguous()[..., None]
    deq_r = qr.float().view(T, -1, 128) * sr[..., None]
    _status_ok(K)
    assert _rel_rms(deq, deq_r) < 3e-2


def test_silu_mul(K):
    torch.manual_seed(4)
    gu = torch.randn(9, 2 * 1024, device=DEV).bfloat16()
    y = K.silu_mul(gu, quant=False)
    torch.testing.assert_close(y.float(), ref.silu_mul(gu).float(), atol=2e-2, rtol=2e-2)
    q, s = K.silu_mul(gu, quant=True)
    qr, sr = ref.silu_mul_quant_fp8(gu)
    deq = q.float().view(9, -1, 128) * s.contiguous()[..., None]
    deq_r = qr.float().view(9, -1, 128) * sr[..., None]
    assert _rel_rms(deq, deq_r) < 3e-2


# ----------------------------------------------------------------------------- rope + KV write + attention
def _mk_cache(K, nb, bs, hkv, d):
    return K.alloc_kv_cache(nb, bs, hkv, d, torch.float8_e4m3fn, DEV)


@pytest.mark.parametrize("D,rot,qknorm", [(128, 128, False), (128, 128, True), (128, 64, True), (64, 64, True), (256, 64, True)])
def test_rope_kv_write(K, D, rot, qknorm):
    torch.manual_seed(5)
    T, Hq, Hkv, bs, nb = 19, 4, 2, 16, 8
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    q = qkv[:, :Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    pos = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(nb * bs, device=DEV)[:T].to(torch.int32)
    slots[3] = -1
    rope = ref.build_rope_cache(rot, 512, 1e6, None, DEV)
    qn = (torch.rand(D, device=DEV) + 0.5).bfloat16() if qknorm else None
    kn = (torch.rand(D, device=DEV) + 0.5).bfloat16() if qknorm else None
    kc, vc = _mk_cache(K, nb, bs, Hkv, D)
    kc_r, vc_r = torch.zeros_like(kc.contiguous()), torch.zeros_like(vc.contiguous())
    q_ref = ref.qk_norm_rope_kv_write(q.clone(), k, v, pos, rope, rot, kc_r, vc_r, slots, 0.5, 0.25, qn, kn, 1e-6, False)
    q_out = K.qk_norm_rope_kv_write(q, k, v, pos, rope, rot, kc, vc, slots, 0.5, 0.25, qn, kn, 1e-6, False)
    _status_ok(K)
    torch.testing.assert_close(q_out.float(), q_ref.float(), atol=3e-2, rtol=3e-2)
    # fp8 rounding can flip one code at ties: compare dequantized values
    assert _rel_rms(kc.float(), kc_r.float()) < 4e-2
    assert _rel_rms(vc.float(), vc_r.float()) < 4e-2


def test_rope_kv_write_prefill_pages(K):
    """Prefill-size batch: V goes through the page-row writer.  Rows cover whole pages in order, a run that starts in
    the middle of a page, a skipped row (slot -1) and a ragged tail."""
    torch.manual_seed(15)
    D, Hq, Hkv, bs, nb = 128, 8, 2, 16, 40
    T = 16 * 20 + 7
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    q = qkv[:, :Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    pos = torch.arange(T, device=DEV, dtype=torch.int32)
    pages = torch.randperm(nb)[:22].tolist()
    slots = []
    for g in range(12):                                   # 12 whole pages in order
        slots += [pages[g] * bs + i for i in range(bs)]
    slots += [pages[12] * bs + 5 + i for i in range(11)]  # a sequence that starts at offset 5 of its page
    slots += [pages[13] * bs + i for i in range(bs)]      # ... and continues: groups of 16 rows straddle pages
    slots += [pages[14] * bs + i for i in range(bs)]
    while len(slots) < T:
        slots.append(pages[15 + (len(slots) // bs) % 6] * bs + len(slots) % bs)
    slots = torch.tensor(slots[:T], device=DEV, dtype=torch.int32)
    slots[40] = -1
    rope = ref.build_rope_cache(D, 512, 1e6, None, DEV)
    kc, vc = _mk_cache(K, nb, bs, Hkv, D)
    kc_r, vc_r = torch.zeros_like(kc.contiguous()), torch.zeros_like(vc.contiguous())
    ref.qk_norm_rope_kv_write(q.clone(), k, v, pos, rope, D, kc_r, vc_r, slots, 0.5, 0.25, None, None, 1e-6, False)
    K.qk_norm_rope_kv_write(q, k, v, pos, rope, D, kc, vc, slots, 0.5, 0.25, None, None, 1e-6, False)
    _status_ok(K)
    assert _rel_rms(kc.float(), kc_r.float()) < 4e-2
    assert _rel_rms(vc.float(), vc_r.float()) < 4e-2
    assert float((vc.float() - vc_r.float()).abs().max()) < 0.6        # no misplaced rows (values are O(1))


def _attention_case(K, D, Hq, Hkv, qlens, ctxs, bs=16, window=None, seed=6, kv_dtype=torch.float8_e4m3fn, oracle_bug=None):
    from atlas_b200.models.batch import ForwardBatch
    torch.manual_seed(seed)
    B = len(qlens)
    tot = [c + q for c, q in zip(ctxs, qlens)]
    nblk = [(t + bs - 1) // bs for t in tot]
    nb = sum(nblk) + 3
    perm = torch.randperm(nb).tolist()
    tables, off = [], 0
    for n in nblk:
        tables.append(perm[off:off + n])
        off += n
    kc, vc = K.alloc_kv_cache(nb, bs, Hkv, D, kv_dtype, DEV)
    # fill the cache through the logical view
    kf = (torch.randn(nb, bs, Hkv, D, device=DEV) * 0.5)
    vf = (torch.randn(nb, bs, Hkv, D, device=DEV) * 0.5)
    kc.copy_(kf.to(kv_dtype))
    vc.copy_(vf.to(kv_dtype))
    toks = [[0] * q for q in qlens]
    fb = ForwardBatch.build(toks, ctxs, tables, bs, device=DEV)
    T = sum(qlens)
    q = (torch.randn(T, Hq, D, device=DEV) * 0.5).bfloat16()
    scale = D ** -0.5
    ks, vs = (0.7, 1.3) if kv_dtype == torch.float8_e4m3fn else (1.0, 1.0)      # a 16-bit cache stores unscaled values
    out = K.paged_attention(q, kc, vc, fb, scale, ks, vs, window)
    if oracle_bug == "mask":              # every row also sees the key after its own position (one more cached token)
        want = ref.paged_attention(q, kc, vc, fb.block_tables, fb.seq_lens + 1, fb.query_start_loc, scale, ks, vs, window)
    elif oracle_bug == "v_scale":
        want = ref.paged_attention(q, kc, vc, fb.block_tables, fb.seq_lens, fb.query_start_loc, scale, ks, 1.0, window)
    elif oracle_bug == "scale":
        want = ref.paged_attention(q, kc, vc, fb.block_tables, fb.seq_lens, fb.query_start_loc, 64 ** -0.5, ks, vs, window)
    else:
        want = ref.paged_attention(q, kc, vc, fb.block_tables, fb.seq_lens, fb.query_start_loc, scale, ks, vs, window)
    _status_ok(K)
    return out, want


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (64, 4, 4), (256, 16, 2), (128, 32, 8)])
def test_attention_bf16_cache(K, D, Hq, Hkv):
    """16-bit KV cache: decode rows (short, page-boundary and split-K lengths), prefill chunks and a mixed batch."""
    out, want = _attention_case(K, D, Hq, Hkv, qlens=[1, 1, 1, 1, 1], ctxs=[1, 15, 16, 200, 3000], kv_dtype=torch.bfloat16)
    assert _rel_rms(out, want) < 1.5e-2
    torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=5e-2)
    out, want = _attention_case(K, D, Hq, Hkv, qlens=[1, 1, 40, 16, 5, 130], ctxs=[33, 700, 0, 48, 100, 77],
                                kv_dtype=torch.bfloat16)
    assert _rel_rms(out, want) < 1.5e-2
    torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=5e-2)


def test_attention_bf16_cache_window_big_pages(K):
    out, want = _attention_case(K, 128, 8, 2, qlens=[1, 1, 50], ctxs=[300, 40, 90], bs=64, window=64, kv_dtype=torch.bfloat16)
    assert _rel_rms(out, want) < 1.5e-2


def test_rope_kv_write_bf16_cache(K):
    torch.manual_seed(16)
    D, Hq, Hkv, bs, nb = 128, 8, 2, 16, 24
    for T in (5, 300):
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
        q = qkv[:, :Hq * D].view(T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        pos = torch.arange(T, device=DEV, dtype=torch.int32)
        slots = torch.randperm(nb * bs, device=DEV)[:T].to(torch.int32)
        rope = ref.build_rope_cache(D, 512, 1e6, None, DEV)
        kc, vc = K.alloc_kv_cache(nb, bs, Hkv, D, torch.bfloat16, DEV)
        kc_r, vc_r = torch.zeros_like(kc.contiguous()), torch.zeros_like(vc.contiguous())
        ref.qk_norm_rope_kv_write(q.clone(), k, v, pos, rope, D, kc_r, vc_r, slots, 1.0, 1.0, None, None, 1e-6, False)
        K.qk_norm_rope_kv_write(q, k, v, pos, rope, D, kc, vc, slots, 1.0, 1.0, None, None, 1e-6, False)
        _status_ok(K)
        assert _rel_rms(kc.float(), kc_r.float()) < 1e-2
        assert _rel_rms(vc.float(), vc_r.float()) < 1e-2


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (64, 4, 4), (256, 16, 2), (128, 32, 8)])
def test_attention_decode(K, D, Hq, Hkv):
    out, want = _attention_case(K, D, Hq, Hkv, qlens=[1, 1, 1, 1, 1], ctxs=[1, 15, 16, 200, 1023])
    assert _rel_rms(out, want) < 2e-2
    torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=5e-2)


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (64, 4, 2), (256, 4, 1)])
def test_attention_prefill_and_mixed(K, D, Hq, Hkv):
    out, want = _attention_case(K, D, Hq, Hkv, qlens=[1, 1, 40, 16, 5, 130], ctxs=[33, 700, 0, 48, 100, 77])
    assert _rel_rms(out, want) < 2e-2
    torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=5e-2)


@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (32, 8), (4, 4), (16, 2), (8, 4)])
def test_attention_prefill_tcgen05(K, Hq, Hkv, monkeypatch):
    """Chunk attention on the tcgen05 path (head_dim 128, 16-token pages, FP8 cache): several GQA group sizes, chunks
    that start inside a context, span many KV tiles and end inside a page; it must agree with the fp32 oracle and with
    the general kernel."""
    qlens, ctxs = [300, 1, 37, 513, 128], [0, 90, 1000, 77, 256]
    out, want = _attention_case(K, 128, Hq, Hkv, qlens=qlens, ctxs=ctxs)
    assert _rel_rms(out, want) < 2e-2
    torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=5e-2)
    monkeypatch.setattr(K, "_TC_PREFILL", False)
    old, _ = _attention_case(K, 128, Hq, Hkv, qlens=qlens, ctxs=ctxs)
    assert _rel_rms(out, old) < 2e-2


def test_attention_sliding_window_and_big_pages(K):
    out, want = _attention_case(K, 128, 8, 2, qlens=[1, 1, 50], ctxs=[300, 40, 90], bs=64, window=64)
    assert _rel_rms(out, want) < 2e-2


def test_fused_gemm_rows_do_not_depend_on_the_batch(K):
    """A row's result must not depend on how many other rows share its launch (decode rows and the same rows inside a
    verify / mixed step go through the same tile plan): every fused epilogue form, 4 rows alone against the same 4 rows
    in front of 16 others, bit for bit."""
    from atlas_b200 import quant as Q
    torch.manual_seed(41)
    H, I = 1024, 2048
    x = torch.randn(20, H, device=DEV).bfloat16()
    xi = torch.randn(20, I, device=DEV).bfloat16()
    w_gu, s_gu = Q.quantize_fp8_block(torch.randn(2 * I, H, device=DEV) * 0.05)
    w_dn, s_dn = Q.quantize_fp8_block(torch.randn(H, I, device=DEV) * 0.05)
    w_q, s_q = Q.quantize_fp8_block(torch.randn(1536, H, device=DEV) * 0.05)
    nw = (torch.randn(H, device=DEV) * 0.2 + 1).bfloat16()
    res = torch.randn(20, H, device=DEV).bfloat16()

    def chain(rows):
        xq, xs = K.quant_fp8(xi[:rows].contiguous())
        r = res[:rows].clone()
        q2, s2, (ss, parts) = K.gemm_fp8_fused(xq, xs, w_dn, s_dn, mode=2, residual=r, norm_w=nw)       # down + norm
        y0 = K.gemm_fp8_fused(q2, s2, w_q, s_q, mode=0, ss_in=(ss, parts, H, 1e-5))                      # next qkv
        q1, s1 = K.gemm_fp8_fused(q2, s2, w_gu, s_gu, mode=1, ss_in=(ss, parts, H, 1e-5))                # next gate|up
        return r, q2.view(torch.uint8), s2, y0, q1.view(torch.uint8), s1

    small, big = chain(4), chain(20)
    _status_ok(K)
    for a, b in zip(small, big):
        assert torch.equal(a, b[:4])


@pytest.mark.parametrize("Hq,Hkv,ctxs,window", [(32, 8, [1, 15, 16, 200, 1023] * 60, None),      # one split per sequence
                                                  (8, 2, [5, 700, 9000], None),                    # split-K + merge kernel
                                                  (16, 2, [300, 40], 64)])
def test_attention_decode_fp8_output(K, Hq, Hkv, ctxs, window):
    """Decode attention that writes FP8 rows + one scale per (row, head) must give exactly what quantising the bf16
    output of the plain kernel gives (the values are rounded to bf16 before they are quantised)."""
    from atlas_b200.models.batch import ForwardBatch
    torch.manual_seed(26)
    D, bs = 128, 16
    B = len(ctxs)
    nblk = [(c + 1 + bs - 1) // bs for c in ctxs]
    nb = sum(nblk) + 3
    perm = torch.randperm(nb).tolist()
    tables, off = [], 0
    for n in nblk:
        tables.append(perm[off:off + n])
        off += n
    kc, vc = K.alloc_kv_cache(nb, bs, Hkv, D, torch.float8_e4m3fn, DEV)
    kc.copy_((torch.randn(nb, bs, Hkv, D, device=DEV) * 0.5).to(torch.float8_e4m3fn))
    vc.copy_((torch.randn(nb, bs, Hkv, D, device=DEV) * 0.5).to(torch.float8_e4m3fn))
    fb = ForwardBatch.build([[0]] * B, ctxs, tables, bs, device=DEV)
    q = (torch.randn(B, Hq, D, device=DEV) * 0.5).bfloat16()
    out = K.paged_attention(q, kc, vc, fb, D ** -0.5, 0.7, 1.3, window)
    got = K.paged_attention_q8(q, kc, vc, fb, D ** -0.5, 0.7, 1.3, window)
    _status_ok(K)
    assert got is not None
    q8, sc = got
    want_q, want_s = K.quant_fp8(out.view(B, Hq * D))
    assert torch.equal(sc, want_s)
    assert torch.equal(q8.view(torch.uint8), want_q.view(torch.uint8))
    # a mixed step (one decode row, one 5-token chunk): decode rows and the chunk meet in the same FP8 buffers
    fb2 = ForwardBatch.build([[0], [0] * 5], [10, 3], [tables[0], tables[1]], bs, device=DEV)
    q2 = (torch.randn(6, Hq, D, device=DEV) * 0.5).bfloat16()
    if window is None and Hq // Hkv in (1, 2, 4, 8):
        out2 = K.paged_attention(q2, kc, vc, fb2, D ** -0.5, 0.7, 1.3, None)
        got2 = K.paged_attention_q8(q2, kc, vc, fb2, D ** -0.5, 0.7, 1.3, None)
        _status_ok(K)
        wq2, ws2 = K.quant_fp8(out2.view(6, Hq * D))
        assert got2 is not None and torch.equal(got2[1], ws2) and torch.equal(got2[0].view(torch.uint8), wq2.view(torch.uint8))
    else:
        # a sliding window is outside the chunk kernel's coverage: the caller is told before anything is launched
        assert K.paged_attention_q8(q2, kc, vc, fb2, D ** -0.5, 1.0, 1.0, 64) is None


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (64, 4, 4), (128, 32, 8)])
def test_attention_decode_e4m3_tiles(K, D, Hq, Hkv):
    """The decode variant that feeds the cached bytes to e4m3 tensor-core tiles (Q and P as two e4m3 terms each) must
    meet the same bounds as the default kernel: single pages, page boundaries, odd page counts, split-K."""
    import ctypes as C
    L = K.lib()
    L.atlas_attn_set_decode_f8.argtypes = [C.c_int]
    L.atlas_attn_set_decode_f8.restype = None
    L.atlas_attn_set_decode_f8(1)
    try:
        out, want = _attention_case(K, D, Hq, Hkv, qlens=[1, 1, 1, 1, 1, 1], ctxs=[1, 15, 16, 40, 200, 1023])
        assert _rel_rms(out, want) < 2e-2
        torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=5e-2)
        out, want = _attention_case(K, D, Hq, Hkv, qlens=[1, 1], ctxs=[5000, 9000])
        assert _rel_rms(out, want) < 2e-2
        out, want = _attention_case(K, D, Hq, Hkv, qlens=[1, 1], ctxs=[300, 40], window=64)
        assert _rel_rms(out, want) < 2e-2
    finally:
        L.atlas_attn_set_decode_f8(0)


def test_attention_prefill_fp8_output(K):
    """The tcgen05 chunk attention kernel with its FP8-output epilogue gives exactly the quantised form of its bf16
    output (pure prefill steps; chunks that start inside a context and end inside a page)."""
    from atlas_b200.models.batch import ForwardBatch
    torch.manual_seed(27)
    D, Hq, Hkv, bs = 128, 16, 4, 16
    qlens, ctxs = [300, 37, 513], [0, 1000, 77]
    nblk = [(c + q + bs - 1) // bs for c, q in zip(ctxs, qlens)]
    nb = sum(nblk) + 3
    perm = torch.randperm(nb).tolist()
    tables, off = [], 0
    for n in nblk:
        tables.append(perm[off:off + n])
        off += n
    kc, vc = K.alloc_kv_cache(nb, bs, Hkv, D, torch.float8_e4m3fn, DEV)
    kc.copy_((torch.randn(nb, bs, Hkv, D, device=DEV) * 0.5).to(torch.float8_e4m3fn))
    vc.copy_((torch.randn(nb, bs, Hkv, D, device=DEV) * 0.5).to(torch.float8_e4m3fn))
    fb = ForwardBatch.build([[0] * q for q in qlens], ctxs, tables, bs, device=DEV)
    T = sum(qlens)
    q = (torch.randn(T, Hq, D, device=DEV) * 0.5).bfloat16()
    out = K.paged_attention(q, kc, vc, fb, D ** -0.5, 0.7, 1.3, None)
    got = K.paged_attention_q8(q, kc, vc, fb, D ** -0.5, 0.7, 1.3, None)
    _status_ok(K)
    assert got is not None
    want_q, want_s = K.quant_fp8(out.view(T, Hq * D))
    assert torch.equal(got[1], want_s)
    assert torch.equal(got[0].view(torch.uint8), want_q.view(torch.uint8))


def test_nvfp4_kv_cache_write_and_attention(K):
    """NVFP4 KV cache: the fused RoPE + cache-write kernel packs K and V (e2m1 + one e4m3 scale per token and 16 dims),
    the result dequantises to the written rows within the format's precision, and decode rows, split-K decode and prefill
    chunks over that cache agree with an fp32 attention over the dequantised contents."""
    from atlas_b200 import quant as Q
    from atlas_b200.models.batch import ForwardBatch
    torch.manual_seed(33)
    D, Hq, Hkv, bs = 128, 8, 2, 16
    ctxs, qlens = [0, 0, 0, 0], [700, 33, 16, 130]
    nblk = [(c + q + 1 + bs - 1) // bs + 1 for c, q in zip(ctxs, qlens)]
    nb = sum(nblk) + 2
    perm = torch.randperm(nb).tolist()
    tables, off = [], 0
    for n in nblk:
        tables.append(perm[off:off + n])
        off += n
    kc, vc = K.alloc_kv_cache(nb, bs, Hkv, D, K.NVFP4_KV, DEV)
    kc16, vc16 = K.alloc_kv_cache(nb, bs, Hkv, D, torch.bfloat16, DEV)
    rope = ref.build_rope_cache(D, 2048, 1e4, None, DEV)
    ks_g, vs_g = 0.02, 0.03                                    # second-level scales of the two tensors
    # ---- prefill: write every prompt row, then attend
    fb = ForwardBatch.build([[0] * q for q in qlens], ctxs, tables, bs, device=DEV)
    T = sum(qlens)
    qkv = (torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV) * 0.6).bfloat16()
    sl = lambda a, n: qkv[:, a * D:(a + n) * D].view(T, n, D)
    q, k, v = sl(0, Hq), sl(Hq, Hkv), sl(Hq + Hkv, Hkv)
    q16 = q.clone()
    qr = K.qk_norm_rope_kv_write(q, k, v, fb.positions, rope, D, kc, vc, fb.slot_mapping, ks_g, vs_g, None, None, 1e-6, False)
    K.qk_norm_rope_kv_write(q16, k, v, fb.positions, rope, D, kc16, vc16, fb.slot_mapping, 1.0, 1.0, None, None, 1e-6, False)
    _status_ok(K)
    Kd, Vd = Q.dequantize_nvfp4_kv(kc, vc, D)
    slots = fb.slot_mapping.long()
    got_k = Kd.reshape(nb * bs, Hkv, D)[slots] * ks_g
    want_k = kc16.reshape(nb * bs, Hkv, D)[slots].float()
    got_v = Vd.reshape(nb * bs, Hkv, D)[slots] * vs_g
    want_v = vc16.reshape(nb * bs, Hkv, D)[slots].float()
    assert _rel_rms(got_k, want_k) < 0.12 and _rel_rms(got_v, want_v) < 0.12        # e2m1: three significant bits at best
    out = K.paged_attention(qr, kc, vc, fb, D ** -0.5, ks_g, vs_g, None)
    want = ref.paged_attention(qr, Kd, Vd, fb.block_tables, fb.seq_lens, fb.query_start_loc, D ** -0.5, ks_g, vs_g, None)
    _status_ok(K)
    assert _rel_rms(out, want) < 2e-2
    # ---- one more token per sequence (decode rows; the 700-token sequence takes the split-K path)
    fb2 = ForwardBatch.build([[0]] * 4, qlens, tables, bs, device=DEV)
    qkv2 = (torch.randn(4, (Hq + 2 * Hkv) * D, device=DEV) * 0.6).bfloat16()
    sl2 = lambda a, n: qkv2[:, a * D:(a + n) * D].view(4, n, D)
    q2 = K.qk_norm_rope_kv_write(sl2(0, Hq), sl2(Hq, Hkv), sl2(Hq + Hkv, Hkv), fb2.positions, rope, D, kc, vc, fb2.slot_mapping,
                                 ks_g, vs_g, None, None, 1e-6, False)
    Kd, Vd = Q.dequantize_nvfp4_kv(kc, vc, D)
    out2 = K.paged_attention(q2, kc, vc, fb2, D ** -0.5, ks_g, vs_g, None)
    want2 = ref.paged_attention(q2, Kd, Vd, fb2.block_tables, fb2.seq_lens, fb2.query_start_loc, D ** -0.5, ks_g, vs_g, None)
    _status_ok(K)
    assert _rel_rms(out2, want2) < 2e-2
    # the earlier rows were not disturbed by the second write (neighbouring tokens share bytes of V)
    got_v2 = Vd.reshape(nb * bs, Hkv, D)[slots] * vs_g
    assert torch.equal(got_v2, got_v)


def test_attention_decode_long_splitk(K):
    out, want = _attention_case(K, 128, 8, 1, qlens=[1, 1], ctxs=[5000, 9000])
    assert _rel_rms(out, want) < 2e-2


@pytest.mark.parametrize("scoring,bias,groups,hashed", [("sigmoid", True, (8, 4), False), ("sqrtsoftplus", True, (0, 0), False),
                                                        ("softmax", True, (0, 0), False), ("sqrtsoftplus", False, (0, 0), True),
                                                        ("sigmoid", False, (4, 2), False)])
def test_moe_route_variants(K, scoring, bias, groups, hashed):
    torch.manual_seed(21)
    T, E, k = 300, 256, 8
    lg = torch.randn(T, E, device=DEV).bfloat16()
    b = (torch.randn(E, device=DEV) * 0.2) if bias else None
    tab = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(500)]).to(torch.int32) if hashed else None
    tok = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32) if hashed else None
    w, ids = K.moe_route(lg, k, True, scoring, b, groups[0], groups[1], 2.5, tab, tok)
    w_r, ids_r = ref.moe_route(lg, k, True, scoring, b, groups[0], groups[1], 2.5, tab, tok)
    # near-ties may order differently in fp32: compare the selected sets through a dense scatter of the weights
    dense = torch.zeros(T, E, device=DEV).scatter_(1, ids.long(), w)
    dense_r = torch.zeros(T, E, device=DEV).scatter_(1, ids_r.long(), w_r)
    assert (ids.long().sort(-1).values == ids_r.long().sort(-1).values).float().mean() > 0.995
    assert float((dense - dense_r).abs().max()) < 0.05 * 2.5
    torch.testing.assert_close(w.sum(-1), torch.full((T,), 2.5, device=DEV), atol=1e-3, rtol=1e-3)


# ----------------------------------------------------------------------------- sampling
def test_argmax_first_index(K):
    torch.manual_seed(7)
    x = torch.randn(6, 151936, device=DEV).bfloat16()
    x[2, 1000] = 50.0
    x[2, 90000] = 50.0
    x[4, :] = 0.0
    got = K.argmax(x)
    assert got.tolist() == ref.argmax_first(x).tolist()
    assert got[2].item() == 1000 and got[4].item() == 0
    assert K.argmax(x.float()).tolist() == got.tolist()


def test_sample_kernel_matches_reference_distribution(K):
    torch.manual_seed(8)
    B, V = 64, 5000
    logits = torch.randn(1, V, device=DEV).repeat(B, 1) * 3
    temp = torch.full((B,), 0.9, device=DEV)
    top_k = torch.full((B,), 40, device=DEV, dtype=torch.int32)
    top_p = torch.full((B,), 0.85, device=DEV)
    min_p = torch.full((B,), 0.02, device=DEV)
    u = torch.rand(B, device=DEV)
    got = K.sample(logits, temp, top_k, top_p, min_p, u)
    # the kept set must be the reference's kept set, and tokens are drawn by inverse CDF in index order
    lf = logits[0].float() / 0.9
    probs = torch.softmax(lf, -1)
    sp, si = torch.sort(probs, descending=True, stable=True)
    keep = torch.arange(V, device=DEV) < 40
    keep &= (sp.cumsum(-1) - sp) < 0.85
    keep &= sp >= 0.02 * sp[0]
    kept_ids = set(si[keep].tolist())
    assert set(got.tolist()) <= kept_ids
    mask = torch.zeros(V, device=DEV, dtype=torch.bool)
    mask[si[keep]] = True
    pk = torch.where(mask, probs, torch.zeros_like(probs))
    cdf = (pk / pk.sum()).cumsum(-1)
    want = torch.searchsorted(cdf, u * (1 - 1e-7), right=True).clamp(max=V - 1)
    agree = (got == want).float().mean().item()
    assert agree > 0.9, agree
    # greedy rows inside a sampling launch
    temp[:8] = 0.0
    got2 = K.sample(logits, temp, top_k, top_p, min_p, u)
    assert got2[:8].tolist() == [int(logits[0].argmax())] * 8


def test_spec_accept(K):
    d = torch.tensor([[1, 2, 3], [4, 5, 6], [7, 8, 9]], device=DEV)
    t = torch.tensor([[1, 2, 3, 0], [4, 0, 6, 1], [0, 8, 9, 2]], device=DEV)
    assert K.spec_accept(d, t).tolist() == [3, 1, 0]


def test_lora_bgmv(K):
    """Per-row adapter update kernel against the fp32 restatement, rows of three kinds (no adapter, slot 1, slot 3)."""
    from atlas_b200.lora import bgmv
    torch.manual_seed(11)
    T, Kd, N = 37, 512, 640
    x = torch.randn(T, Kd, device=DEV).bfloat16()
    slots = torch.tensor([0, 1, 3] * 12 + [1], device=DEV, dtype=torch.int64)
    ads = {1: (torch.randn(8, Kd, device=DEV) * 0.1, torch.randn(N, 8, device=DEV) * 0.1),
           3: (torch.randn(16, Kd, device=DEV) * 0.1, torch.randn(N, 16, device=DEV) * 0.1)}
    sc = {1: 2.0, 3: 0.5}
    y0 = torch.randn(T, 1024, device=DEV).bfloat16()
    y = y0.clone()
    K.lora_bgmv(x, slots, ads, sc, y, 128, N)
    ads16 = {s: (a.bfloat16(), b.bfloat16()) for s, (a, b) in ads.items()}
    want = y0.float()
    want[:, 128:128 + N] += bgmv(x, ads16, slots, sc)
    _status_ok(K)
    assert torch.equal(y[:, :128], y0[:, :128]) and torch.equal(y[:, 128 + N:], y0[:, 128 + N:])
    assert torch.equal(y[slots == 0], y0[slots == 0])
    torch.testing.assert_close(y.float(), want, atol=3e-2, rtol=2e-2)


# ----------------------------------------------------------------------------------------------------- fused GEMM epilogues
@pytest.mark.parametrize("M,I,Kd", [(128, 1024, 512), (300, 2048, 1024), (5, 256, 256)])
def test_gemm_fused_swiglu_quant(K, M, I, Kd):
    """gate|up GEMM whose epilogue applies SiLU * mul and quantises to FP8 groups: against fp32 silu(gate) * up of the
    dequantised operands, and against the unfused kernel sequence."""
    torch.manual_seed(5)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = torch.randn(2 * I, Kd, device=DEV) * 0.05
    wq, ws = Q.quantize_fp8_block(w)
    xq, xs = K.quant_fp8(x)
    q, s = K.gemm_fp8_fused(xq, xs, wq, ws, mode=1)
    gu = Q.fp8_block_gemm_ref(xq, xs.contiguous(), wq, ws, out_dtype=torch.float32)
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    _status_ok(K)
    deq = (q.float().view(M, -1, 128) * s.contiguous()[..., None]).view(M, I)
    assert _rel_rms(deq, want) < 4e-2
    q2, s2 = K.silu_mul(K.gemm_fp8_block(xq, xs, wq, ws), quant=True)
    deq2 = (q2.float().view(M, -1, 128) * s2.contiguous()[..., None]).view(M, I)
    assert _rel_rms(deq, deq2) < 3e-2


@pytest.mark.parametrize("M,N,Kd,plus_one", [(128, 1024, 512, False), (300, 2048, 4096, True), (3, 512, 2048, False)])
def test_gemm_fused_residual_norm_quant_and_deferred_factor(K, M, N, Kd, plus_one):
    """Row-parallel-style GEMM whose epilogue adds the residual, multiplies by the norm weight and quantises, leaving the
    1/rms factor to the consumer GEMM: the pair must equal GEMM -> residual add -> RMSNorm -> GEMM in fp32."""
    torch.manual_seed(6)
    eps = 1e-6
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = torch.randn(N, Kd, device=DEV) * 0.05
    resid = torch.randn(M, N, device=DEV).bfloat16()
    norm_w = (torch.randn(N, device=DEV) * 0.2 + (0.0 if plus_one else 1.0)).bfloat16()
    w2 = torch.randn(384, N, device=DEV) * 0.05
    wq, ws = Q.quantize_fp8_block(w)
    w2q, w2s = Q.quantize_fp8_block(w2)
    xq, xs = K.quant_fp8(x)
    res = resid.clone()
    q, s, (ss, tiles) = K.gemm_fp8_fused(xq, xs, wq, ws, mode=2, residual=res, norm_w=norm_w, plus_one=plus_one)
    y = K.gemm_fp8_fused(q, s, w2q, w2s, mode=0, ss_in=(ss, tiles, N, eps))
    _status_ok(K)
    h = Q.fp8_block_gemm_ref(xq, xs.contiguous(), wq, ws, out_dtype=torch.float32) + resid.float()
    assert _rel_rms(res, h) < 1e-2
    weff = norm_w.float() + (1.0 if plus_one else 0.0)
    normed = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * weff
    want = normed @ Q.dequantize_fp8_block(w2q, w2s).float().t()
    assert _rel_rms(y, want) < 4e-2
    rstd = torch.rsqrt(ss[:, :M].sum(0) / N + eps)
    assert _rel_rms(rstd, torch.rsqrt(h.pow(2).mean(-1) + eps)) < 1e-2
    # the deferred factor also composes with the SwiGLU epilogue
    wg = torch.randn(512, N, device=DEV) * 0.05
    wgq, wgs = Q.quantize_fp8_block(wg)
    qa, sa = K.gemm_fp8_fused(q, s, wgq, wgs, mode=1, ss_in=(ss, tiles, N, eps))
    gu = normed @ Q.dequantize_fp8_block(wgq, wgs).float().t()
    want_a = torch.nn.functional.silu(gu[:, :256]) * gu[:, 256:]
    deq = (qa.float().view(M, -1, 128) * sa.contiguous()[..., None]).view(M, 256)
    _status_ok(K)
    assert _rel_rms(deq, want_a) < 6e-2


@pytest.mark.parametrize("T", [7, 300])
def test_rotated_kv_write_and_head_rotation(K, T):
    """The "turbo8" cache write: q / k / v heads go through the orthonormal 128-point Walsh-Hadamard transform after
    RoPE (prefill-size batches too, which otherwise send V through the page-row writer), against the matrix form; and
    the in-place rotation of an attention output, which is its own inverse."""
    torch.manual_seed(21)
    D, Hq, Hkv, bs, nb = 128, 8, 2, 16, 24
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qkv[:, 5::128] *= 20.0                                 # an outlier channel in every head
    q = qkv[:, :Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    pos = torch.arange(T, device=DEV, dtype=torch.int32)
    slots = torch.randperm(nb * bs, device=DEV)[:T].to(torch.int32)
    rope = ref.build_rope_cache(D, 512, 1e6, None, DEV)
    qn = (torch.rand(D, device=DEV) + 0.5).bfloat16()
    kc, vc = _mk_cache(K, nb, bs, Hkv, D)
    kc_r, vc_r = torch.zeros_like(kc.contiguous()), torch.zeros_like(vc.contiguous())
    q_ref = ref.qk_norm_rope_kv_write(q.clone(), k, v, pos, rope, D, kc_r, vc_r, slots, 0.5, 0.25, qn, qn, 1e-6, False, rotate=True)
    q_out = K.qk_norm_rope_kv_write(q, k, v, pos, rope, D, kc, vc, slots, 0.5, 0.25, qn, qn, 1e-6, False, rotate=True)
    _status_ok(K)
    assert _rel_rms(q_out, q_ref) < 1e-2
    assert _rel_rms(kc.float(), kc_r.float()) < 4e-2 and _rel_rms(vc.float(), vc_r.float()) < 4e-2
    x = torch.randn(T, Hq, D, device=DEV).bfloat16()
    y = K.wht_d128(x.clone())
    _status_ok(K)
    assert _rel_rms(y, ref.head_rotate(x)) < 5e-3
    assert _rel_rms(K.wht_d128(y.clone()), x) < 8e-3       # an involution up to bf16 rounding


def test_oracle_bounds_reject_plausibly_wrong_kernels(K):
    """The bounds the numerics tests use must be able to fail: each case compares a CORRECT kernel result with an oracle
    that carries one realistic kernel bug (a weight-scale block skipped, the causal mask off by one key, the value scale
    dropped, the softmax scale of another head size) and must land outside the bound the real test applies."""
    torch.manual_seed(3)
    # FP8 block-scaled GEMM: one 128-wide K block of one 128-row weight block uses a neighbour's scale
    M, N, K_ = 256, 512, 1024
    x = torch.randn(M, K_, device=DEV).bfloat16()
    wq, ws = Q.quantize_fp8_block(torch.randn(N, K_, device=DEV) * 0.05 * (1 + torch.arange(K_, device=DEV) // 128))
    xq, xs = K.quant_fp8(x)
    out = K.gemm_fp8_block(xq, xs, wq, ws)
    _status_ok(K)
    good = Q.fp8_block_gemm_ref(xq, xs.contiguous(), wq, ws, out_dtype=torch.float32)
    bad_ws = ws.clone()
    bad_ws[1, 3] = ws[1, 2]
    bad = Q.fp8_block_gemm_ref(xq, xs.contiguous(), wq, bad_ws, out_dtype=torch.float32)
    assert _rel_rms(out, good) < 5e-3 < _rel_rms(out, bad)
    # paged attention (decode rows and a prefill chunk): mask off by one key / value scale dropped / wrong softmax scale
    D, Hq, Hkv = 128, 8, 2
    out, want = _attention_case(K, D, Hq, Hkv, qlens=[1, 1, 40, 130], ctxs=[33, 700, 0, 77])
    assert _rel_rms(out, want) < 2e-2
    for mutate in ("mask", "v_scale", "scale"):
        wrong = _attention_case(K, D, Hq, Hkv, qlens=[1, 1, 40, 130], ctxs=[33, 700, 0, 77], oracle_bug=mutate)[1]
        assert _rel_rms(out, wrong) > 2e-2, mutate
