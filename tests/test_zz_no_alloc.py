"""The allocation-free RMSNorm backward must agree with the regular entry point.

Some users of the library cannot allocate device memory where they need this op (fixed memory
pools, serving loops that forbid allocation stalls, embedders that own all device memory), so
``axb_rmsnorm_bwd_noalloc`` keeps its fp32 partial-sum workspace in a device array inside the
library.  This test calls it through its exported C symbol, twice in a row (the workspace is
shared between calls and keeps stale contents), and compares with ``axb_rmsnorm_bwd`` run on a
workspace the test allocates.  It lives in a file that pytest collects last so that a failure
here cannot hide any other test under ``-x``.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_D = 8192


def _entry_points():
    from axlearn_b200.ops import cuda_ops

    lib = cuda_ops.lib()
    fn = lib.axb_rmsnorm_bwd_noalloc
    vp = ctypes.c_void_p
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_int64, ctypes.c_int, vp]
    fn.restype = ctypes.c_int
    return lib, fn


def _inputs(rows, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    dy = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    dres = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    scale = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    return x, scale, rstd, dy, dres


def _regular(lib, x, scale, rstd, dy, dres):
    rows, d = x.shape
    ctas = lib.axb_rmsnorm_bwd_ctas(rows)
    partial = torch.empty(ctas, d, device="cuda")
    dx = torch.empty_like(x)
    ds16 = torch.empty(d, device="cuda", dtype=torch.bfloat16)
    ds32 = torch.empty(d, device="cuda")
    rc = lib.axb_rmsnorm_bwd(x.data_ptr(), scale.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dres.data_ptr(),
                             dx.data_ptr(), partial.data_ptr(), ds16.data_ptr(), ds32.data_ptr(), rows, d,
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return dx, ds16, ds32


def _noalloc(fn, x, scale, rstd, dy, dres):
    rows, d = x.shape
    dx = torch.empty_like(x)
    ds16 = torch.empty(d, device="cuda", dtype=torch.bfloat16)
    ds32 = torch.empty(d, device="cuda")
    rc = fn(x.data_ptr(), scale.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dres.data_ptr(), dx.data_ptr(),
            ds16.data_ptr(), ds32.data_ptr(), rows, d, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return dx, ds16, ds32


def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row():
    lib, fn = _entry_points()
    # Two different problems back to back: the second call finds the first one's partial sums
    # (for a wider D and more CTAs) still in the shared workspace and must not be affected.
    for rows, d, seed in [(3000, 4096, 0), (77, 1024, 1)]:
        args = _inputs(rows, d, seed)
        want = _regular(lib, *args)
        got = _noalloc(fn, *args)
        torch.cuda.synchronize()
        for w, g in zip(want, got):
            err = (w.float() - g.float()).abs().max().item()
            scale = w.float().abs().max().item() + 1e-6
            assert err / scale < 2e-2, (rows, d, err, scale)
            assert torch.equal(w, g)  # same math, same summation order


def _fp32_reference(x, scale, rstd, dy, dres):
    """RMSNorm backward written out in fp32 PyTorch: y = x * rstd * scale."""
    xf, dyf, sf = x.float(), dy.float(), scale.float()
    xhat = xf * rstd[:, None]
    g = dyf * sf
    dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    return dx, (dyf * xhat).sum(0)


def _assert_close(got, want, atol, rtol, what):
    diff = (got.float() - want.float()).abs()
    bound = atol + rtol * want.float().abs()
    assert bool((diff <= bound).all()), (what, diff.max().item())


@pytest.mark.parametrize("rows,d,with_dres,with_f32,with_bf16", [
    (513, 4096, True, True, True),
    (64, MAX_D, True, True, False),   # the largest width the built-in workspace holds
    (300, 1024, False, False, True),  # no residual gradient, no fp32 scale gradient
    (40, 512, False, True, False),
])
def test_noalloc_against_fp32_pytorch(rows, d, with_dres, with_f32, with_bf16):
    _, fn = _entry_points()
    x, scale, rstd, dy, dres = _inputs(rows, d, 3)
    dx = torch.empty_like(x)
    ds16 = torch.full((d,), 7.0, device="cuda", dtype=torch.bfloat16)
    ds32 = torch.full((d,), 7.0, device="cuda")
    for _ in range(2):  # the second call reuses the workspace the first one left behind
        rc = fn(x.data_ptr(), scale.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dres.data_ptr() if with_dres else None,
                dx.data_ptr(), ds16.data_ptr() if with_bf16 else None, ds32.data_ptr() if with_f32 else None, rows, d,
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0
    torch.cuda.synchronize()
    want_dx, want_ds = _fp32_reference(x, scale, rstd, dy, dres if with_dres else None)
    _assert_close(dx, want_dx, 2e-2, 2e-2, "dx")
    if with_f32:
        _assert_close(ds32, want_ds, 1e-2 * want_ds.abs().max().item(), 1e-3, "dscale fp32")
    else:
        assert torch.all(ds32 == 7.0)  # a null output is not written
    if with_bf16:
        _assert_close(ds16, want_ds, 2e-2 * want_ds.abs().max().item(), 2e-2, "dscale bf16")
    else:
        assert torch.all(ds16 == 7.0)


def test_noalloc_with_no_rows_zeroes_the_scale_gradient():
    _, fn = _entry_points()
    d = 256
    x, scale, rstd, dy, dres = _inputs(1, d, 4)
    ds32 = torch.full((d,), 7.0, device="cuda")
    rc = fn(x.data_ptr(), scale.data_ptr(), rstd.data_ptr(), dy.data_ptr(), None, x.data_ptr(), None, ds32.data_ptr(),
            0, d, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.all(ds32 == 0.0)


def test_noalloc_rejects_sizes_beyond_its_workspace():
    _, fn = _entry_points()
    d = MAX_D + 8
    x, scale, rstd, dy, dres = _inputs(4, d, 2)
    dx = torch.full_like(x, 7.0)
    rc = fn(x.data_ptr(), scale.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dres.data_ptr(), dx.data_ptr(),
            None, None, 4, d, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == -20
    assert torch.all(dx == 7.0)  # nothing was launched
