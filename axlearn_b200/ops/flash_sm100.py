"""Launch wrappers of the tcgen05 flash-attention kernels (``csrc/flash_fwd.cu``,
``csrc/flash_bwd.cu``)."""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from axlearn_b200.ops import cuda_ops

import os

c_void_p, c_int, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_configured = False
FORWARD_VARIANT = os.environ.get("AXB200_FLASH_FWD", "v3")
# "fused": one kernel, five GEMMs per tile pair, dQ reduced with fp32 vector atomics (not
# bit-reproducible).  "split": the deterministic dK/dV + dQ kernel pair (causal / full masks only).
BACKWARD_VARIANT = os.environ.get("AXB200_FLASH_BWD", "fused")


def _lib():
    global _configured
    h = cuda_ops.lib()
    if not _configured:
        h.axb_flash_fwd.argtypes = [c_void_p] * 5 + [c_int] * 6 + [c_float, c_int, c_void_p, c_void_p]
        h.axb_flash_fwd.restype = c_int
        h.axb_flash_fwd_v2.argtypes = h.axb_flash_fwd.argtypes
        h.axb_flash_fwd_v2.restype = c_int
        h.axb_flash_bwd.argtypes = [c_void_p] * 10 + [c_int] * 6 + [c_float, c_int, c_void_p, c_void_p]
        h.axb_flash_bwd.restype = c_int
        h.axb_flash_fwd_v3.argtypes = [c_void_p] * 8 + [c_int] * 6 + [c_float, c_int, c_int, c_float, c_void_p, c_void_p]
        h.axb_flash_fwd_v3.restype = c_int
        h.axb_seg_tile_ranges.argtypes = [c_void_p] * 3 + [c_int] * 3 + [c_void_p]
        h.axb_seg_tile_ranges.restype = c_int
        h.axb_flash_bwd_fused.argtypes = ([c_void_p] * 15 + [c_int] * 6 + [c_float, c_int, c_int, c_float, c_void_p,
                                                                           c_void_p])
        h.axb_flash_bwd_fused.restype = c_int
        _configured = True
    return h


def segment_tile_ranges(q_seg: torch.Tensor, k_seg: torch.Tensor) -> torch.Tensor:
    """int32 ``[B, ceil(T/128), 2]``: for every 128-row query tile the range of 128-key tiles that
    hold a key of one of the tile's segments (the kernels skip everything outside)."""
    b, t = q_seg.shape
    s = k_seg.shape[1]
    ranges = torch.empty((b, (t + 127) // 128, 2), dtype=torch.int32, device=q_seg.device)
    rc = _lib().axb_seg_tile_ranges(q_seg.data_ptr(), k_seg.data_ptr(), ranges.data_ptr(), b, t, s,
                                    cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_seg_tile_ranges")  # pylint: disable=protected-access
    return ranges


def forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool, scale: float,
            q_seg: Optional[torch.Tensor] = None, k_seg: Optional[torch.Tensor] = None,
            ranges: Optional[torch.Tensor] = None, window: Optional[int] = None,
            logit_cap: Optional[float] = None):
    """q ``[B, T, N, H]``, k/v ``[B, S, Nkv, H]`` bf16 contiguous -> (out, lse ``[B, N, T]``).

    ``q_seg [B, T]`` / ``k_seg [B, S]`` (int32): a key is visible only to queries with the same
    id; ``ranges`` comes from ``segment_tile_ranges``.  ``window``: keys more than ``window``
    positions before the query are hidden.  ``logit_cap``: scores become ``cap * tanh(s / cap)``.
    """
    b, t, n, h = q.shape
    s, nkv = k.shape[1], k.shape[2]
    out = torch.empty_like(q)
    lse = torch.empty((b, n, t), dtype=torch.float32, device=q.device)
    h_lib = _lib()
    general = q_seg is not None or window is not None or logit_cap is not None
    status = cuda_ops.status_word(q.device).data_ptr()
    if FORWARD_VARIANT == "v3" or general:
        # Two query tiles per CTA, eight softmax warps per tile, in-kernel masks.
        rc = h_lib.axb_flash_fwd_v3(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
            cuda_ops._p(q_seg), cuda_ops._p(k_seg), cuda_ops._p(ranges),  # pylint: disable=protected-access
            b, t, s, n, nkv, h, scale, 1 if causal else 0, -1 if window is None else int(window),
            0.0 if logit_cap is None else float(logit_cap), status, cuda_ops._stream())  # pylint: disable=protected-access
    else:
        # "v2" (four softmax warps per tile) and "v1" (one query tile, probabilities through
        # shared memory) are kept as cross-checks.
        fn = h_lib.axb_flash_fwd if FORWARD_VARIANT == "v1" else h_lib.axb_flash_fwd_v2
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                b, t, s, n, nkv, h, scale, 1 if causal else 0, status, cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_flash_fwd")  # pylint: disable=protected-access
    return out, lse


def backward(q, k, v, out, lse, dout, *, causal: bool, scale: float, q_seg=None, k_seg=None, k_ranges=None,
             window: Optional[int] = None, logit_cap: Optional[float] = None, variant: Optional[str] = None):
    """Gradients ``(dq, dk, dv)``.  ``k_ranges`` is ``segment_tile_ranges(k_seg, q_seg)`` (indexed by
    key tile)."""
    b, t, n, h = q.shape
    s, nkv = k.shape[1], k.shape[2]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    general = q_seg is not None or window is not None or logit_cap is not None
    status = cuda_ops.status_word(q.device).data_ptr()
    if (variant or BACKWARD_VARIANT) == "fused" or general:
        tp = (t + 127) // 128 * 128
        lse2 = torch.empty((b, n, tp), dtype=torch.float32, device=q.device)
        delta = torch.empty_like(lse2)
        dq_acc = torch.empty((b, n, tp, h), dtype=torch.float32, device=q.device)
        rc = _lib().axb_flash_bwd_fused(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            lse2.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            cuda_ops._p(q_seg), cuda_ops._p(k_seg), cuda_ops._p(k_ranges),  # pylint: disable=protected-access
            b, t, s, n, nkv, h, scale, 1 if causal else 0, -1 if window is None else int(window),
            0.0 if logit_cap is None else float(logit_cap), status, cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_flash_bwd_fused")  # pylint: disable=protected-access
        cuda_ops.launch_count += 2
        return dq, dk, dv
    delta = torch.empty_like(lse)
    rc = _lib().axb_flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                              lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                              b, t, s, n, nkv, h, scale, 1 if causal else 0, status,
                              cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_flash_bwd")  # pylint: disable=protected-access
    cuda_ops.launch_count += 2
    return dq, dk, dv
