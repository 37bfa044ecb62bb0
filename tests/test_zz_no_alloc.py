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
