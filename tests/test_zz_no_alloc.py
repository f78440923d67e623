"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the point where they launch kernels (an embedded
plugin whose host owns the allocator, a loop with a no-allocation rule).  For them the library carries its split-K
scratch as a fixed array; this test checks that variant against the ordinary entry point, twice in a row (the array
keeps the first call's contents, so the second call shows that stale data does not leak into results), and that
an over-sized request is refused.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,splits", [(128, 5), (64, 3), (128, 1)])
def test_noalloc_decode_matches_regular_entry_twice(D, splits):
    from atlas_b200.models.batch import ForwardBatch
    from atlas_b200.ops import cuda as K
    K.load()
    lib = K.lib()
    vp, ll, i, f = C.c_void_p, C.c_longlong, C.c_int, C.c_float
    fn = lib.atlas_attn_decode_noalloc
    fn.argtypes = [vp, ll, vp, ll, vp, vp, vp, i, vp, vp, i, f, f, f, i, i, i, i, i, i, vp, vp]
    fn.restype = i
    dev = "cuda"
    Hq, Hkv, bs = 8, 2, 16
    for round_, ctxs in enumerate(([700, 33, 1500], [90, 2047, 640])):
        torch.manual_seed(40 + round_)
        B = len(ctxs)
        nblk = [(c + 1 + bs - 1) // bs for c in ctxs]
        nb = sum(nblk) + 2
        perm = torch.randperm(nb).tolist()
        tables, off = [], 0
        for n in nblk:
            tables.append(perm[off:off + n])
            off += n
        kc, vc = K.alloc_kv_cache(nb, bs, Hkv, D, torch.float8_e4m3fn, dev)
        kc.copy_((torch.randn(nb, bs, Hkv, D, device=dev) * 0.5).to(torch.float8_e4m3fn))
        vc.copy_((torch.randn(nb, bs, Hkv, D, device=dev) * 0.5).to(torch.float8_e4m3fn))
        fb = ForwardBatch.build([[0]] * B, ctxs, tables, bs, device=dev)
        q = (torch.randn(B, Hq, D, device=dev) * 0.5).bfloat16()
        want = K.paged_attention(q, kc, vc, fb, D ** -0.5, 0.7, 1.3, None)       # regular entry (allocates its scratch)
        d = K._dev(q)
        out = torch.empty_like(want)
        torch.cuda.synchronize()
        rc = fn(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, kc.data_ptr(), vc.data_ptr(), fb.block_tables.data_ptr(),
                fb.block_tables.stride(0), fb.seq_lens.data_ptr(), fb.query_start_loc.data_ptr(), B, D ** -0.5, 0.7, 1.3,
                Hq, Hkv, D, bs, 0, splits, K._status_ptr[d], torch.cuda.current_stream().cuda_stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert K.check_status() == 0
        torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=5e-2)
    # beyond the compiled-in scratch: refused with the documented code, nothing launched
    rc = fn(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, kc.data_ptr(), vc.data_ptr(), fb.block_tables.data_ptr(),
            fb.block_tables.stride(0), fb.seq_lens.data_ptr(), fb.query_start_loc.data_ptr(), 4096, D ** -0.5, 0.7, 1.3,
            Hq, Hkv, D, bs, 0, 64, K._status_ptr[d], torch.cuda.current_stream().cuda_stream)
    assert rc == -100
    # unsupported shapes are refused before the size test
    rc = fn(q.data_ptr(), q.stride(0), out.data_ptr(), Hq * D, kc.data_ptr(), vc.data_ptr(), fb.block_tables.data_ptr(),
            fb.block_tables.stride(0), fb.seq_lens.data_ptr(), fb.query_start_loc.data_ptr(), B, D ** -0.5, 0.7, 1.3,
            0, Hkv, D, bs, 0, 2, K._status_ptr[d], torch.cuda.current_stream().cuda_stream)
    assert rc == -1
