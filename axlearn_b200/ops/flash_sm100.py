"""Launch wrappers of the tcgen05 flash-attention kernels (``csrc/flash_fwd.cu``,
``csrc/flash_bwd.cu``)."""

from __future__ import annotations

import ctypes

import torch

from axlearn_b200.ops import cuda_ops

import os

c_void_p, c_int, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_configured = False
FORWARD_VARIANT = os.environ.get("AXB200_FLASH_FWD", "v2")


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
        _configured = True
    return h


def forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool, scale: float):
    """q ``[B, T, N, H]``, k/v ``[B, S, Nkv, H]`` bf16 contiguous -> (out, lse ``[B, N, T]``)."""
    b, t, n, h = q.shape
    s, nkv = k.shape[1], k.shape[2]
    out = torch.empty_like(q)
    lse = torch.empty((b, n, t), dtype=torch.float32, device=q.device)
    h_lib = _lib()
    # "v2" (two query tiles per CTA, probabilities in tensor memory) is the default;
    # "v1" (one query tile, probabilities through shared memory) is kept as a cross-check.
    fn = h_lib.axb_flash_fwd if FORWARD_VARIANT == "v1" else h_lib.axb_flash_fwd_v2
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                              b, t, s, n, nkv, h, scale, 1 if causal else 0,
                              cuda_ops.status_word(q.device).data_ptr(), cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_flash_fwd")  # pylint: disable=protected-access
    return out, lse


def backward(q, k, v, out, lse, dout, *, causal: bool, scale: float):
    b, t, n, h = q.shape
    s, nkv = k.shape[1], k.shape[2]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty_like(lse)
    rc = _lib().axb_flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                              lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                              b, t, s, n, nkv, h, scale, 1 if causal else 0,
                              cuda_ops.status_word(q.device).data_ptr(), cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_flash_bwd")  # pylint: disable=protected-access
    cuda_ops.launch_count += 2
    return dq, dk, dv
