"""Block-scaled fp8 kernels against the torch emulation (same fp8 rounding, fp32 reference sums)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _emulated(fn):
    from axlearn_b200.ops import dispatch

    with dispatch.use_reference_ops():
        return fn()


@pytest.mark.parametrize("e5m2", [False, True])
def test_quantisers_match_emulation(e5m2):
    from axlearn_b200.ops import fp8_ops

    torch.manual_seed(0)
    x = (torch.randn(300, 512, device="cuda") * torch.logspace(-3, 3, 300, device="cuda")[:, None]).bfloat16()
    q, s = fp8_ops.quantize_rows(x, e5m2=e5m2)
    qr, sr = _emulated(lambda: fp8_ops.quantize_rows(x, e5m2=e5m2))
    assert torch.allclose(s, sr, rtol=1e-6)
    assert (q.float() - qr.float()).abs().max() <= 0.13 * qr.float().abs().max()   # at most one fp8 step apart
    assert (q.float() != qr.float()).float().mean() < 0.02
    for transpose in (False, True):
        q, s = fp8_ops.quantize_blocks(x, transpose=transpose, e5m2=e5m2)
        qr, sr = _emulated(lambda: fp8_ops.quantize_blocks(x, transpose=transpose, e5m2=e5m2))
        assert q.shape == qr.shape and torch.allclose(s, sr, rtol=1e-6)
        assert (q.float() != qr.float()).float().mean() < 0.02


@pytest.mark.parametrize("m,n,k", [(256, 256, 512), (300, 384, 1024), (4096, 1024, 2048)])
@pytest.mark.parametrize("a_gran", [1, 128])
def test_gemm_fp8_matches_dequantised_reference(m, n, k, a_gran):
    from axlearn_b200.ops import cuda_ops, fp8_ops

    torch.manual_seed(1)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = (torch.randn(n, k, device="cuda") * 0.1).bfloat16()
    aq, sa = fp8_ops.quantize_rows(a) if a_gran == 1 else fp8_ops.quantize_blocks(a)
    bq, sb = fp8_ops.quantize_blocks(b, e5m2=True)
    out = fp8_ops.gemm_fp8(aq, bq, sa, sb, a_gran=a_gran, out_dtype=torch.float32)
    ref = fp8_ops.dequantize(aq, sa, row_gran=a_gran) @ fp8_ops.dequantize(bq, sb, row_gran=128).t()
    torch.cuda.synchronize()
    cuda_ops.check_status()
    assert (out - ref).abs().max() < 2e-3 * ref.abs().max(), (out - ref).abs().max() / ref.abs().max()
    out16 = fp8_ops.gemm_fp8(aq, bq, sa, sb, a_gran=a_gran)
    assert (out16.float() - ref).abs().max() < 1e-2 * ref.abs().max()


def test_fp8_linear_matches_emulation_and_tracks_bf16():
    from axlearn_b200.ops import cuda_ops, fp8_ops

    torch.manual_seed(2)
    x = torch.randn(4, 256, 512, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(512, 768, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    g = torch.randn(4, 256, 768, device="cuda").bfloat16()

    def run():
        y = fp8_ops.fp8_linear(x, w)
        return (y,) + torch.autograd.grad(y, [x, w], g)

    before = cuda_ops.launch_count
    got = run()
    assert cuda_ops.launch_count - before >= 9   # 3 GEMMs + 6 quantiser launches
    emu = _emulated(run)
    torch.cuda.synchronize()
    cuda_ops.check_status()
    yr = x.float() @ w.float()
    exact = (yr,) + torch.autograd.grad(yr, [x, w], g.float())
    for a, e, r in zip(got, emu, exact):
        assert (a.float() - e.float()).abs().max() < 2e-2 * e.float().abs().max()
        assert (a.float() - r).abs().max() < 0.1 * r.abs().max()
