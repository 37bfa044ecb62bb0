"""Block-scaled fp8 matmuls: quantisers, the tcgen05 GEMM (``csrc/gemm_fp8.cu``) and a linear op
with fp8 forward / data-gradient / weight-gradient GEMMs.

Recipe (per GEMM, all scales fp32, blocks of 128 along the contraction dim):

* forward ``y = x @ w``:   x rows in 1x128 blocks (e4m3), w in 128x128 blocks (e4m3);
* data gradient ``dx = dy @ w^T``: dy rows in 1x128 blocks (e5m2), the same w blocks;
* weight gradient ``dw = x^T @ dy``: x and dy in 128x128 blocks (e4m3 / e5m2), contraction over
  tokens.

Every function has a torch emulation (quantise -> dequantise -> fp32 matmul) that is used on CPU
and as the oracle for the kernels: both paths round to exactly the same fp8 values, so they differ
only by fp32 summation order.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from axlearn_b200.ops import cuda_ops

c_void_p, c_int, c_int64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
_configured = False
E4M3_MAX, E5M2_MAX = 448.0, 57344.0


def _lib():
    global _configured
    h = cuda_ops.lib()
    if not _configured:
        h.axb_gemm_fp8.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64,
                                   c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        h.axb_quantize_rows.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p]
        h.axb_quantize_blocks.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int,
                                          c_void_p]
        for f in (h.axb_gemm_fp8, h.axb_quantize_rows, h.axb_quantize_blocks):
            f.restype = c_int
        _configured = True
    return h


def _dtype(e5m2: bool):
    return torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn


def kernels_available(*tensors: torch.Tensor) -> bool:
    from axlearn_b200.ops import dispatch

    return all(t.is_cuda for t in tensors) and not dispatch._flags.force_reference  # pylint: disable=protected-access


# ------------------------------------------------------------------------------ quantisers
def quantize_rows(x: torch.Tensor, *, e5m2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """x ``[R, C]`` bf16 -> (fp8 ``[R, C]``, scales ``[R, C / 128]``): one scale per row and 128
    columns, ``scale = amax / max_normal``."""
    r, c = x.shape
    assert c % 128 == 0
    if kernels_available(x) and x.dtype == torch.bfloat16:
        x = x.contiguous()
        q = torch.empty((r, c), dtype=_dtype(e5m2), device=x.device)
        s = torch.empty((r, c // 128), dtype=torch.float32, device=x.device)
        rc = _lib().axb_quantize_rows(x.data_ptr(), c, q.data_ptr(), c, s.data_ptr(), r, c, 1 if e5m2 else 0,
                                      cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_quantize_rows")  # pylint: disable=protected-access
        return q, s
    xf = x.float().reshape(r, c // 128, 128)
    amax = xf.abs().amax(dim=-1)
    s = torch.where(amax > 0, amax / (E5M2_MAX if e5m2 else E4M3_MAX), torch.ones_like(amax))
    q = (xf / s[..., None]).to(_dtype(e5m2)).reshape(r, c)
    return q, s


def quantize_blocks(x: torch.Tensor, *, transpose: bool = False, e5m2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """x ``[R, C]`` bf16 -> 128x128-block-scaled fp8.  ``transpose``: returns ``x^T`` quantised
    (``[C, R]``, scales ``[C/128, R/128]``) without materialising a bf16 transpose."""
    r, c = x.shape
    rb, cb = (r + 127) // 128, (c + 127) // 128
    if kernels_available(x) and x.dtype == torch.bfloat16:
        x = x.contiguous()
        shape, sshape = ((c, r), (cb, rb)) if transpose else ((r, c), (rb, cb))
        q = torch.empty(shape, dtype=_dtype(e5m2), device=x.device)
        s = torch.empty(sshape, dtype=torch.float32, device=x.device)
        rc = _lib().axb_quantize_blocks(x.data_ptr(), c, q.data_ptr(), shape[1], s.data_ptr(), r, c,
                                        1 if transpose else 0, 1 if e5m2 else 0, cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_quantize_blocks")  # pylint: disable=protected-access
        return q, s
    xf = torch.zeros((rb * 128, cb * 128), dtype=torch.float32, device=x.device)
    xf[:r, :c] = x.float()
    blocks = xf.reshape(rb, 128, cb, 128)
    amax = blocks.abs().amax(dim=(1, 3))
    s = torch.where(amax > 0, amax / (E5M2_MAX if e5m2 else E4M3_MAX), torch.ones_like(amax))
    q = (blocks / s[:, None, :, None]).reshape(rb * 128, cb * 128)[:r, :c].to(_dtype(e5m2))
    if transpose:
        return q.t().contiguous(), s.t().contiguous()
    return q, s


def dequantize(q: torch.Tensor, s: torch.Tensor, *, row_gran: int) -> torch.Tensor:
    """fp32 matrix from fp8 ``[R, C]`` and scales ``[ceil(R / row_gran), C / 128]``."""
    r, c = q.shape
    rows = torch.arange(r, device=q.device) // row_gran
    cols = torch.arange(c, device=q.device) // 128
    return q.float() * s[rows][:, cols]


# ------------------------------------------------------------------------------ GEMM
def gemm_fp8(a: torch.Tensor, b: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor, *, a_gran: int = 1,
             out_dtype: torch.dtype = torch.bfloat16, max_ctas: int = 0) -> torch.Tensor:
    """``C[M, N] = sum_kb (a[:, kb] @ b[:, kb]^T) * sa[m / a_gran, kb] * sb[n / 128, kb]`` for fp8
    ``a [M, K]``, ``b [N, K]`` (K contiguous), K and N multiples of 128."""
    m, k = a.shape
    n = b.shape[0]
    assert b.shape[1] == k and k % 128 == 0 and n % 128 == 0, (a.shape, b.shape)
    assert sa.shape == ((m + a_gran - 1) // a_gran, k // 128) and sb.shape == (n // 128, k // 128), (sa.shape, sb.shape)
    if kernels_available(a, b):
        a, b, sa, sb = a.contiguous(), b.contiguous(), sa.contiguous(), sb.contiguous()
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
        fmt = lambda t: 1 if t.dtype == torch.float8_e5m2 else 0
        if max_ctas == 0 and cuda_ops.COMM_RESERVED_SMS:
            max_ctas = max(8, cuda_ops._sm_count(a.device) - cuda_ops.COMM_RESERVED_SMS)  # pylint: disable=protected-access
        rc = _lib().axb_gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), sa.data_ptr(), sb.data_ptr(), m, n, k,
                                 k, k, n, fmt(a), fmt(b), a_gran, 1 if out_dtype == torch.float32 else 0,
                                 cuda_ops.status_word(a.device).data_ptr(), max_ctas, cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_gemm_fp8")  # pylint: disable=protected-access
        return out
    return (dequantize(a, sa, row_gran=a_gran) @ dequantize(b, sb, row_gran=128).t()).to(out_dtype)


# ------------------------------------------------------------------------------ linear
def supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the fp8 linear covers: contraction and output dims multiples of 128, and a token
    count that is a multiple of 128 (it is the contraction dim of the weight gradient)."""
    tokens = x.numel() // x.shape[-1]
    return x.shape[-1] % 128 == 0 and w.shape[1] % 128 == 0 and tokens % 128 == 0 and tokens > 0


class _Fp8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):  # x [..., K] bf16, w [K, N]
        x2 = x.reshape(-1, x.shape[-1])
        xq, sx = quantize_rows(x2)
        wq_t, sw_t = quantize_blocks(w, transpose=True)                      # [N, K], [N/128, K/128]
        ctx.save_for_backward(x2, w)
        return gemm_fp8(xq, wq_t, sx, sw_t, a_gran=1, out_dtype=x.dtype).reshape(x.shape[:-1] + (w.shape[1],))

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq, sdy = quantize_rows(dy2, e5m2=True)
            wq, sw = quantize_blocks(w)                                       # [K, N], [K/128, N/128]
            dx = gemm_fp8(dyq, wq, sdy, sw, a_gran=1, out_dtype=dy.dtype).reshape(x2.shape)
        if ctx.needs_input_grad[1]:
            xq_t, sx_t = quantize_blocks(x2, transpose=True)                  # [K, M]
            dyq_t, sdy_t = quantize_blocks(dy2, transpose=True, e5m2=True)    # [N, M]
            dw = gemm_fp8(xq_t, dyq_t, sx_t, sdy_t, a_gran=128, out_dtype=w.dtype)
        return (None if dx is None else dx.reshape(dy.shape[:-1] + (x2.shape[1],))), dw


def fp8_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x[..., K] @ w[K, N]`` with all three GEMMs in block-scaled fp8 (see the module docstring)."""
    return _Fp8Linear.apply(x, w.contiguous() if not w.is_contiguous() else w)
