"""Tensor-parallel reductions over peer memory instead of library all-reduces.

A reduction over a tensor-parallel group is a one-shot all-reduce on NVLink: every rank stores its
partial into its slot of every peer's staging buffer and raises a flag; every rank then sums the
slots in a fixed order (``ops/decode_ops.OneShotAllReduce``: bounded flag waits that report
through the device status word).  For a row-parallel linear the store half is the epilogue of the
GEMM itself (``csrc/gemm_2cta.cu`` ``rs_mode = 1``: every finished tile leaves the tensor core for
all peers' staging with TMA stores while the next tile is computed), so the only extra launch is
the sum.  Counterpart of the ``psum`` XLA inserts around the reference's tensor-parallel einsums
(axlearn/common/attention.py:3803-3850 for the shardings).

Two staging sites per tensor size alternate, which is enough: a peer cannot start the use after
next before this rank has finished reading the current one (it needs this rank's next push first).
Every rank of the group must issue the same sequence of reductions, which SPMD code does.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

ENABLED = os.environ.get("AXB200_TP_PEER", "1") != "0"
# Staging is 2 sites x world slots per tensor size; sizes whose staging would exceed this stay
# on the library path.
MAX_STAGING_BYTES = int(os.environ.get("AXB200_TP_PEER_MAX_BYTES", str(2 << 30)))

_pools: dict = {}


class _Pool:
    def __init__(self, numel: int, group, device):
        from axlearn_b200.ops import decode_ops

        self.reducer = decode_ops.OneShotAllReduce(numel, 2, group=group, device=device)
        self.uses = 0

    def site(self) -> int:
        site = self.uses % 2
        if site == 0:
            self.reducer.begin_step()      # one epoch per pair of uses: each site once per epoch
        self.uses += 1
        return site


def usable(x: torch.Tensor, group, world: int) -> bool:
    if not ENABLED or group is None or world < 2 or world > 8:
        return False
    if not (x.is_cuda and x.dtype == torch.bfloat16) or x.numel() % 8 or x.numel() == 0:
        return False
    return 2 * world * x.numel() * 2 <= MAX_STAGING_BYTES


def _pool(numel: int, group, device) -> _Pool:
    key = (id(group), numel, device.index)
    pool = _pools.get(key)
    if pool is None:
        pool = _pools[key] = _Pool(numel, group, device)
    return pool


def reset() -> None:
    """Forgets every pool (a new process group invalidates their symmetric buffers)."""
    _pools.clear()


def all_reduce(x: torch.Tensor, group) -> torch.Tensor:
    """Sum of ``x`` over ``group`` (a new tensor)."""
    x = x.contiguous()
    pool = _pool(x.numel(), group, x.device)
    site = pool.site()
    pool.reducer.push(x.reshape(-1), site)
    return pool.reducer.finish(site).view(x.shape)


def gemm_all_reduce(a: torch.Tensor, b: torch.Tensor, group) -> torch.Tensor:
    """``sum over group of (a [M, K] @ b [K, N])``; the GEMM's epilogue does the stores."""
    m, n = a.shape[0], b.shape[1]
    pool = _pool(m * n, group, a.device)
    site = pool.site()
    if n % 32 == 0:
        pool.reducer.gemm_push(a, b, site)
    else:
        from axlearn_b200.ops import cuda_ops

        pool.reducer.push(cuda_ops.gemm(a, b).reshape(-1), site)
    return pool.reducer.finish(site).view(m, n)


class _PsumPeer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return all_reduce(x, group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _PsumGradPeer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return all_reduce(g, ctx.group), None


class _RowParallelLinear(torch.autograd.Function):
    """``psum(x @ w)`` with the stores of the reduction in the GEMM epilogue; the gradients are
    those of a plain linear (the incoming gradient is already the same on every rank)."""

    @staticmethod
    def forward(ctx, x, w, group):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = gemm_all_reduce(x2, w, group)
        return y.view(x.shape[:-1] + (w.shape[1],))

    @staticmethod
    def backward(ctx, dy):
        from axlearn_b200.ops import cuda_ops

        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = cuda_ops.gemm(dy2, w.t()).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            if w.stride(0) == 1 and w.stride(1) != 1:      # a transposed view of a row-major [N, K] tensor
                dw = cuda_ops.gemm(dy2.t(), x2).t()
            else:
                dw = cuda_ops.gemm(x2.t(), dy2)
        return dx, dw, None


def psum(x: torch.Tensor, group) -> torch.Tensor:
    return _PsumPeer.apply(x, group)


def psum_grad(x: torch.Tensor, group) -> torch.Tensor:
    return _PsumGradPeer.apply(x, group)


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, group, world: int) -> Optional[torch.Tensor]:
    """``psum(x @ w)`` on the fused path, or None when it does not apply (the caller then runs the
    product and the reduction separately)."""
    from axlearn_b200.common import remat

    if remat.active() is not None:       # kept products are handled by the plain linear
        return None
    if w.dtype != torch.bfloat16 or x.shape[-1] % 8 or w.shape[1] % 8:
        return None
    from axlearn_b200.ops import cuda_ops

    if x.is_cuda and cuda_ops.carries_gather(w):
        # The weight is also storage-sharded by the fused FSDP runtime, whose linear gathers it
        # and scatters its gradient from inside its own GEMMs: that linear runs, and the
        # reduction over the tensor-parallel group follows as a separate peer all-reduce.
        return None
    rows = x.numel() // x.shape[-1]
    if not (x.is_cuda and x.dtype == torch.bfloat16 and ENABLED and group is not None and 2 <= world <= 8):
        return None
    if 2 * world * rows * w.shape[1] * 2 > MAX_STAGING_BYTES or rows * w.shape[1] % 8:
        return None
    return _RowParallelLinear.apply(x, w, group)
