"""Token dispatch / combine for mixture-of-experts layers (``csrc/moe.cu``) with autograd.

``dest [T, K]`` (int32) gives, for every (token, choice), the row of the flat expert buffer
``[R, M]`` it occupies, or -1 when the assignment was dropped.  Rows are unique, so dispatch is a
gather through the inverse map and needs no zero-fill pass or atomics.

* ``dispatch(x [T, M], dest, num_rows) -> [R, M]``
* ``combine(y [R, M], weight [T, K] fp32, dest) -> [T, M]`` = ``sum_k weight[t, k] * y[dest[t, k]]``

The backward passes are the same kernels with the roles swapped (plus ``row_dots`` for the gate
weights).  Non-bf16 / CPU inputs use an index_add / gather formulation in torch, which is also
the oracle in tests.
"""

from __future__ import annotations

import ctypes

import torch

from axlearn_b200.ops import cuda_ops

c_void_p, c_int, c_int64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
_configured = False


def _lib():
    global _configured
    h = cuda_ops.lib()
    if not _configured:
        h.axb_moe_gather_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]
        h.axb_moe_combine_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
        h.axb_moe_row_dots.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
        for f in (h.axb_moe_gather_rows, h.axb_moe_combine_rows, h.axb_moe_row_dots):
            f.restype = c_int
        _configured = True
    return h


def _use_kernels(t: torch.Tensor) -> bool:
    from axlearn_b200.ops import dispatch as op_dispatch

    return (t.is_cuda and t.dtype == torch.bfloat16 and t.shape[-1] % 8 == 0
            and not op_dispatch._flags.force_reference)  # pylint: disable=protected-access


def inverse_pairs(dest: torch.Tensor, num_rows: int) -> torch.Tensor:
    """``inv[r]`` = flat (token * K + choice) index occupying expert-buffer row r, -1 if empty."""
    flat = dest.reshape(-1).long()
    inv = torch.full((num_rows + 1,), -1, dtype=torch.int32, device=dest.device)
    pair = torch.arange(flat.numel(), dtype=torch.int32, device=dest.device)
    inv[torch.where(flat >= 0, flat, torch.full_like(flat, num_rows))] = pair
    return inv[:num_rows]


def _gather_rows(src, idx, scale, rows):
    out = torch.empty((rows, src.shape[1]), dtype=src.dtype, device=src.device)
    rc = _lib().axb_moe_gather_rows(src.data_ptr(), idx.data_ptr(), None if scale is None else scale.data_ptr(),
                                    out.data_ptr(), rows, src.shape[1], cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_moe_gather_rows")  # pylint: disable=protected-access
    return out


def _combine_rows(y, dest, w, tokens, k):
    out = torch.empty((tokens, y.shape[1]), dtype=y.dtype, device=y.device)
    rc = _lib().axb_moe_combine_rows(y.data_ptr(), dest.data_ptr(), None if w is None else w.data_ptr(),
                                     out.data_ptr(), tokens, k, y.shape[1], cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_moe_combine_rows")  # pylint: disable=protected-access
    return out


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dest, inv, num_rows):
        k = dest.shape[1]
        token_of_row = torch.where(inv >= 0, inv // k, inv)
        ctx.save_for_backward(dest)
        ctx.tokens = x.shape[0]
        return _gather_rows(x.contiguous(), token_of_row.contiguous(), None, num_rows)

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        return _combine_rows(g.contiguous(), dest, None, ctx.tokens, dest.shape[1]), None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, weight, dest, inv):
        y = y.contiguous()
        weight = weight.float().contiguous()
        ctx.save_for_backward(y, weight, dest, inv)
        return _combine_rows(y, dest, weight, dest.shape[0], dest.shape[1])

    @staticmethod
    def backward(ctx, g):
        y, weight, dest, inv = ctx.saved_tensors
        g = g.contiguous()
        k = dest.shape[1]
        token_of_row = torch.where(inv >= 0, inv // k, inv).contiguous()
        w_of_row = weight.reshape(-1)[inv.clamp(min=0).long()].contiguous()
        dy = _gather_rows(g, token_of_row, w_of_row, y.shape[0])
        dw = torch.empty(dest.shape, dtype=torch.float32, device=g.device)
        rc = _lib().axb_moe_row_dots(g.data_ptr(), y.data_ptr(), dest.data_ptr(), dw.data_ptr(), dest.shape[0], k,
                                     y.shape[1], cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_moe_row_dots")  # pylint: disable=protected-access
        return dy, dw, None, None


def dispatch(x: torch.Tensor, dest: torch.Tensor, num_rows: int) -> torch.Tensor:
    """``x [T, M] -> [num_rows, M]``; rows nobody maps to are zero."""
    if _use_kernels(x):
        dest = dest.to(torch.int32).contiguous()
        return _Dispatch.apply(x, dest, inverse_pairs(dest, num_rows), num_rows)
    t, k = dest.shape
    flat = dest.reshape(-1).long()
    flat = torch.where(flat >= 0, flat, torch.full_like(flat, num_rows))
    src = torch.arange(t, device=x.device).repeat_interleave(k)
    buf = torch.zeros((num_rows + 1, x.shape[1]), dtype=x.dtype, device=x.device)
    return buf.index_add(0, flat, x[src])[:-1]


def combine(y: torch.Tensor, weight: torch.Tensor, dest: torch.Tensor) -> torch.Tensor:
    """``y [R, M], weight [T, K], dest [T, K] -> [T, M]``."""
    if _use_kernels(y):
        dest = dest.to(torch.int32).contiguous()
        return _Combine.apply(y, weight, dest, inverse_pairs(dest, y.shape[0]))
    t, k = dest.shape
    flat = dest.reshape(-1).long()
    padded = torch.cat([y, y.new_zeros((1, y.shape[1]))], dim=0)
    gathered = padded[torch.where(flat >= 0, flat, torch.full_like(flat, y.shape[0]))].reshape(t, k, -1)
    return (gathered.float() * weight[..., None].float()).sum(dim=1).to(y.dtype)
