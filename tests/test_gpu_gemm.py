"""tcgen05 GEMM vs an fp32 PyTorch reference, over operand layouts, shapes and outputs."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float()


def _close(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 256, 256), (384, 512, 192), (200, 264, 72), (1024, 4096, 1024), (2048, 11008, 512)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(m, n, k, a_t, b_t):
    from axlearn_b200.ops import cuda_ops

    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn(k, m, device=dev).bfloat16().t() if a_t else torch.randn(m, k, device=dev).bfloat16()
    b = torch.randn(n, k, device=dev).bfloat16().t() if b_t else torch.randn(k, n, device=dev).bfloat16()
    out = cuda_ops.gemm(a, b)
    torch.cuda.synchronize()
    cuda_ops.check_status()
    _close(out, _ref(a, b))


def test_gemm_fp32_out_and_accumulate():
    from axlearn_b200.ops import cuda_ops

    torch.manual_seed(1)
    a = torch.randn(256, 320, device="cuda").bfloat16()
    b = torch.randn(320, 384, device="cuda").bfloat16()
    out = cuda_ops.gemm(a, b, out_dtype=torch.float32)
    _close(out, _ref(a, b), tol=1e-3)
    base = torch.randn(256, 384, device="cuda")
    acc = base.clone()
    cuda_ops.gemm(a, b, out=acc, accumulate=True)
    _close(acc, base + _ref(a, b), tol=1e-3)
    cuda_ops.check_status()


def test_linear_autograd_matches_reference():
    from axlearn_b200.ops import cuda_ops

    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device="cuda").bfloat16().requires_grad_()
    w = torch.randn(256, 512, device="cuda").bfloat16().requires_grad_()
    wt = torch.randn(384, 256, device="cuda").bfloat16().requires_grad_()  # used as x @ wt.t()
    y = cuda_ops.linear(x, w)
    z = cuda_ops.linear(x, wt.t())
    g1, g2 = torch.randn_like(y), torch.randn_like(z)
    (y * g1).sum().backward(retain_graph=True)
    (z * g2).sum().backward()
    xf, wf, wtf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_(), wt.detach().float().requires_grad_()
    yr, zr = xf @ wf, xf @ wtf.t()
    ((yr * g1.float()).sum() + (zr * g2.float()).sum()).backward()
    _close(y, yr)
    _close(z, zr)
    _close(x.grad, xf.grad)
    _close(w.grad, wf.grad)
    _close(wt.grad, wtf.grad)
    cuda_ops.check_status()


def test_gemm_deterministic():
    from axlearn_b200.ops import cuda_ops

    a = torch.randn(512, 1024, device="cuda").bfloat16()
    b = torch.randn(1024, 768, device="cuda").bfloat16()
    assert torch.equal(cuda_ops.gemm(a, b), cuda_ops.gemm(a, b))


@pytest.mark.parametrize("m,n,k", [(64, 1536, 4096), (16, 2752, 4096), (8, 4096, 1376), (128, 4096, 11008), (1, 1536, 512),
                                   (8, 12288, 4096), (16, 22016, 4096), (48, 4096, 4096), (8, 32768, 4096), (5, 9504, 2112)])
@pytest.mark.parametrize("b_t", [False, True])
def test_skinny_gemm_split_k(m, n, k, b_t):
    """Decode-shaped problems (one row block): 64-column tiles, split over K or cut into equal
    runs of (tile, k-block) units per SM (stream-K) where the plan says so; bf16 and fp32 outputs,
    with and without accumulation, repeated to exercise the counters."""
    from axlearn_b200.ops import cuda_ops

    torch.manual_seed(2)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16().t() if b_t else torch.randn(k, n, device="cuda").bfloat16()
    ref = _ref(a, b)
    for _ in range(3):
        _close(cuda_ops.gemm(a, b), ref)
    _close(cuda_ops.gemm(a, b, out_dtype=torch.float32), ref, tol=1e-3)
    base = torch.randn(m, n, device="cuda").bfloat16()
    acc = base.clone()
    cuda_ops.gemm(a, b, out=acc, accumulate=True)
    _close(acc, base.float() + ref)
    torch.cuda.synchronize()
    cuda_ops.check_status()
    if n * 2 <= 148 * 64 and k >= 4096:
        assert cuda_ops.lib().axb_gemm_splitk_plan(m, n, k) > 1


def _close_elementwise(out, ref, atol, rtol):
    """Per-element ``|out - ref| <= atol + rtol * |ref|`` (an error confined to small outputs or one
    tile edge cannot hide behind the largest value)."""
    diff = (out.float() - ref).abs()
    bound = atol + rtol * ref.abs()
    bad = diff > bound
    assert not bad.any(), f"{int(bad.sum())} elements off; worst {diff.max().item():.4g} at {tuple(torch.nonzero(bad)[0].tolist())}"


@pytest.mark.parametrize("variant", ["1cta", "2cta"])
@pytest.mark.parametrize("m,n,k", [(2048, 2048, 512), (4096, 4096, 256), (2304, 2816, 328), (2056, 2064, 72)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_large_gemm_variants_per_element(variant, m, n, k, a_t, b_t, monkeypatch):
    from axlearn_b200.ops import cuda_ops

    monkeypatch.setattr(cuda_ops, "GEMM_VARIANT", variant)
    torch.manual_seed(2)
    a = torch.randn(k, m, device="cuda").bfloat16().t() if a_t else torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16().t() if b_t else torch.randn(k, n, device="cuda").bfloat16()
    out = cuda_ops.gemm(a, b)
    torch.cuda.synchronize()
    cuda_ops.check_status()
    # bf16 rounding of the result (2^-8 relative) plus fp32 accumulation noise.
    _close_elementwise(out, _ref(a, b), atol=0.05 * (k / 256) ** 0.5, rtol=1e-2)


def test_cta_pair_gemm_fp32_out_and_accumulate(monkeypatch):
    from axlearn_b200.ops import cuda_ops

    monkeypatch.setattr(cuda_ops, "GEMM_VARIANT", "2cta")
    torch.manual_seed(3)
    a = torch.randn(2048, 320, device="cuda").bfloat16()
    b = torch.randn(320, 2304, device="cuda").bfloat16()
    ref = _ref(a, b)
    out = cuda_ops.gemm(a, b, out_dtype=torch.float32)
    _close_elementwise(out, ref, atol=1e-3, rtol=1e-4)
    base = torch.randn(2048, 2304, device="cuda")
    acc = base.clone()
    cuda_ops.gemm(a, b, out=acc, accumulate=True)
    _close_elementwise(acc, base + ref, atol=1e-3, rtol=1e-4)
    base16 = torch.randn(2048, 2304, device="cuda").bfloat16()
    acc16 = base16.clone()
    cuda_ops.gemm(a, b, out=acc16, accumulate=True)
    _close_elementwise(acc16, base16.float() + ref, atol=0.15, rtol=1e-2)
    # A strided output (a column block of a wider matrix) goes through the same store path.
    wide = torch.zeros(2048, 4608, device="cuda", dtype=torch.bfloat16)
    cuda_ops.gemm(a, b, out=wide[:, 2304:])
    _close_elementwise(wide[:, 2304:], ref, atol=0.08, rtol=1e-2)
    assert wide[:, :2304].abs().max().item() == 0
    cuda_ops.check_status()


def test_gemm_shape_fuzz(monkeypatch):
    """Seeded random shapes, including sizes that are no multiple of any tile dimension."""
    import random

    from axlearn_b200.ops import cuda_ops

    rng = random.Random(1234)
    for case in range(24):
        variant = "2cta" if case % 2 else "1cta"
        monkeypatch.setattr(cuda_ops, "GEMM_VARIANT", variant)
        m = rng.choice([8 * rng.randint(1, 40), 128 * rng.randint(1, 24), 8 * rng.randint(250, 400)])
        n = rng.choice([8 * rng.randint(1, 40), 128 * rng.randint(1, 24), 8 * rng.randint(250, 400)])
        k = 8 * rng.randint(1, 96)
        a_t, b_t = rng.random() < 0.5, rng.random() < 0.5
        a = torch.randn(k, m, device="cuda").bfloat16().t() if a_t else torch.randn(m, k, device="cuda").bfloat16()
        b = torch.randn(n, k, device="cuda").bfloat16().t() if b_t else torch.randn(k, n, device="cuda").bfloat16()
        out = cuda_ops.gemm(a, b)
        torch.cuda.synchronize()
        cuda_ops.check_status()
        _close_elementwise(out, _ref(a, b), atol=0.05 * max(1.0, (k / 256) ** 0.5), rtol=1e-2)
