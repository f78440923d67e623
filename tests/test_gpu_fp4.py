"""NVFP4 x NVFP4 GEMM on the block-scaled tensor cores and the activation quantiser, against fp32 restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def K():
    from atlas_b200.ops import cuda as K
    K.load()
    return K


def _rel_rms(a, b):
    return float((a.float() - b.float()).pow(2).mean().sqrt() / b.float().pow(2).mean().sqrt().clamp_min(1e-12))


@pytest.mark.parametrize("M,Kd", [(5, 64), (300, 1024), (128, 4096 + 32)])
def test_quant_nvfp4_activations(K, M, Kd):
    from atlas_b200 import quant as Q
    from atlas_b200.ops import cuda_fp4 as F
    torch.manual_seed(1)
    x = (torch.randn(M, Kd, device=DEV) * torch.rand(M, 1, device=DEV) * 4).bfloat16()
    x[0, :16] = 0
    q, sf, rs = F.quant_nvfp4(x)
    assert K.check_status() == 0
    back = F.dequant(q, sf, rs, M, Kd)
    # 4-bit values with a shared scale per 16: ~9 % relative RMS on Gaussian data, and never off by more than half a
    # quantisation step of the group (step <= amax16 / 3 -> error <= amax16 / 6, plus the e4m3 rounding of the scale)
    assert _rel_rms(back, x) < 0.12
    amax16 = x.float().view(M, -1, 16).abs().amax(-1, keepdim=True)
    err = (back - x.float()).view(M, -1, 16).abs()
    assert bool((err <= amax16 / 6 * 1.15 + 1e-6).all())
    # the per-row scale is amax / (6 * 448) and the scale factors use the full e4m3 range
    torch.testing.assert_close(rs, x.float().abs().amax(-1) / (6 * 448), rtol=1e-5, atol=0)
    s = F.sf_from_atoms(sf, M, Kd).view(torch.float8_e4m3fn).float()
    assert float(s.max()) <= 448 and float(s.amax(-1).min()) >= 416


@pytest.mark.parametrize("M,N,Kd", [(128, 128, 256), (128, 256, 1024), (300, 384, 1024 + 64), (1000, 1152, 4096), (64, 128, 64),
                                    (2048, 2560, 1024 + 64), (2500, 2560, 512)])        # the last two take the 256-wide tile
def test_gemm_nvfp4_w4a4(K, M, N, Kd):
    from atlas_b200 import quant as Q
    from atlas_b200.ops import cuda_fp4 as F
    torch.manual_seed(2)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = torch.randn(N, Kd, device=DEV) * 0.05
    wq, ws, wg = Q.quantize_nvfp4(w)
    wsf = F.sf_atoms(ws)
    col = wg.expand(N).contiguous()
    xq, xsf, xrs = F.quant_nvfp4(x)
    out = F.gemm_w4a4(xq, xsf, xrs, wq, wsf, col)
    torch.cuda.synchronize()
    assert K.check_status() == 0
    a = F.dequant(xq, xsf, xrs, M, Kd)
    b = Q.dequantize_nvfp4(wq, ws, wg)
    want = a @ b.t()
    assert _rel_rms(out, want) < 5e-3, _rel_rms(out, want)
    # and against the unquantised product: two 4-bit operands
    assert _rel_rms(out, x.float() @ w.t()) < 0.2


def test_quant_kernel_matches_restatement(K):
    from atlas_b200.ops import cuda_fp4 as F
    from atlas_b200.ops import reference as ref
    torch.manual_seed(3)
    x = (torch.randn(64, 2048, device=DEV) * 3).bfloat16()
    q, sf, rs = F.quant_nvfp4(x)
    got = F.dequant(q, sf, rs, 64, 2048)
    want = ref.quant_nvfp4_rowwise(x)
    # same algorithm; single values may differ by one code where x / scale sits on a rounding boundary
    assert float((got != want).float().mean()) < 2e-3
    assert _rel_rms(got, want) < 2e-2


def test_linear_w4a4_through_ops(K, monkeypatch):
    """An NVFP4 LinearWeight through ``ops.linear`` with activation quantisation on: GPU kernel path vs the fp32
    restatement of the same two quantisations."""
    from atlas_b200 import ops
    from atlas_b200.ops import LinearWeight
    torch.manual_seed(4)
    monkeypatch.setattr(ops, "NVFP4_ACTIVATIONS", True)
    w = LinearWeight.from_dense((torch.randn(768, 1024, device=DEV) * 0.05).bfloat16(), "nvfp4")
    x = torch.randn(200, 1024, device=DEV).bfloat16()
    got = ops.linear(x, w)
    ops.FORCE_REFERENCE = True
    try:
        want = ops.linear(x, w)
    finally:
        ops.FORCE_REFERENCE = False
    assert K.check_status() == 0
    assert _rel_rms(got, want) < 1e-2
