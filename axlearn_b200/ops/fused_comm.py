"""Fused compute+collective ops over NVLink peer memory.

* ``ag_gemm``: ``x @ W`` where ``W`` is stored as one contiguous row-slab per rank (FSDP).  A few
  CTAs of the GEMM kernel pull the peers' slabs into a local full-size buffer with bulk
  asynchronous copies while the remaining CTAs start on the rank's own slab; tiles that need a
  remote slab wait on a per-slab flag (bounded).  This is the reference's "all-gather the bf16
  parameters, then matmul" (axlearn/common/attention.py:3803-3850 shardings, collectives
  inserted by XLA) as one kernel.
* ``gemm_rs``: weight-gradient GEMM whose epilogue stores each output row into the staging slot
  of the rank that owns it (a peer store when the owner is another GPU); ``reduce_slots`` then
  sums the per-rank partials in a fixed order.  Together they replace "matmul, then
  reduce-scatter".

Pointers to peer memory come from ``axlearn_b200.parallel.symm`` (real ranks) or are plain local
tensors in single-GPU tests.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from axlearn_b200.ops import cuda_ops

MAX_PEERS = 8
c_void_p, c_int, c_int64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64


class FusedParams(ctypes.Structure):
    """Host mirror of ``axb::FusedParams`` (csrc/gemm.cu)."""

    _fields_ = [
        ("ag_src", c_void_p * MAX_PEERS),
        ("ag_dst", c_void_p),
        ("ag_flags", c_void_p),
        ("ag_cnt", c_void_p),
        ("ag_shard_bytes", c_int64),
        ("ag_world", c_int),
        ("ag_rank", c_int),
        ("ag_epoch", c_int),
        ("ag_copy_ctas", c_int),
        ("ag_along_k", c_int),
        ("ag_shard_extent", c_int),
        ("rs_dst", c_void_p * MAX_PEERS),
        ("rs_world", c_int),
        ("rs_rank", c_int),
        ("rs_rows_per_rank", c_int),
    ]


_configured = False


def _lib():
    global _configured
    h = cuda_ops.lib()
    if not _configured:
        h.axb_gemm_bf16_fused.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64,
                                          c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]
        h.axb_gemm_bf16_fused.restype = c_int
        h.axb_signal_peers.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p]
        h.axb_signal_peers.restype = c_int
        h.axb_wait_flags.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p]
        h.axb_wait_flags.restype = c_int
        h.axb_reduce_slots_ctas.argtypes = [c_int64]
        h.axb_reduce_slots_ctas.restype = c_int
        h.axb_reduce_slots.argtypes = [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p]
        h.axb_reduce_slots.restype = c_int
        _configured = True
    return h


class GatherState:
    """Per-operand scratch of ``ag_gemm``: the full-size buffer, slab flags, arrival counters
    and the epoch that distinguishes successive gathers into the same buffer."""

    def __init__(self, full_shape: Sequence[int], world: int, device):
        self.full = torch.empty(tuple(full_shape), dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros(world, dtype=torch.int32, device=device)
        self.cnt = torch.zeros(world, dtype=torch.int32, device=device)
        self.epoch = 0


def ag_gemm(x: torch.Tensor, *, shard_ptrs: Sequence[int], state: GatherState, rank: int,
            weight_is_nk: bool = False, copy_ctas: int = 8, out: Optional[torch.Tensor] = None,
            max_ctas: int = 0) -> torch.Tensor:
    """``x[M, K] @ W`` with W gathered inside the kernel.

    ``shard_ptrs[r]`` is the address of rank r's slab (``W[r*rows/R:(r+1)*rows/R]``), its own for
    ``r == rank``.  ``state.full`` has W's full shape: ``[K, N]`` (slabs split the contraction
    dim) or, with ``weight_is_nk``, ``[N, K]`` used as ``x @ W^T`` (slabs split the output dim).
    After the call ``state.full`` holds the whole of W and can be reused (e.g. by the backward).
    """
    world = len(shard_ptrs)
    full = state.full
    rows, cols = full.shape
    x2 = x.reshape(-1, x.shape[-1])
    m, k = x2.shape
    n = rows if weight_is_nk else cols
    assert (cols if weight_is_nk else rows) == k, (full.shape, x2.shape)
    assert rows % world == 0
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    state.epoch += 1
    fp = FusedParams()
    for r, p in enumerate(shard_ptrs):
        fp.ag_src[r] = p
    fp.ag_dst = full.data_ptr()
    fp.ag_flags = state.flags.data_ptr()
    fp.ag_cnt = state.cnt.data_ptr()
    fp.ag_shard_bytes = (rows // world) * cols * 2
    fp.ag_world, fp.ag_rank, fp.ag_epoch, fp.ag_copy_ctas = world, rank, state.epoch, copy_ctas
    fp.ag_along_k = 0 if weight_is_nk else 1
    fp.ag_shard_extent = rows // world
    fp.rs_world = 1
    x2c, a_mn, lda = cuda_ops._operand(x2, 1)  # pylint: disable=protected-access
    # B as the kernel sees it: [K, N]. weight_is_nk: stored [N, K] -> K-major B (b_mn = 0).
    b_mn, ldb = (0, cols) if weight_is_nk else (1, cols)
    cap = max_ctas or (cuda_ops._sm_count(x.device) - cuda_ops.COMM_RESERVED_SMS)  # pylint: disable=protected-access
    rc = _lib().axb_gemm_bf16_fused(x2c.data_ptr(), full.data_ptr(), out.data_ptr(), m, n, k, lda, ldb,
                                    out.stride(0), a_mn, b_mn, cuda_ops.status_word(x.device).data_ptr(), cap,
                                    ctypes.addressof(fp), cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_gemm_bf16_fused(ag)")  # pylint: disable=protected-access
    return out.reshape(x.shape[:-1] + (n,))


def gemm_rs(a: torch.Tensor, b: torch.Tensor, *, staging_ptrs: Sequence[int], rank: int, max_ctas: int = 0) -> None:
    """``C = a[M, K] @ b[K, N]`` whose rows are scattered: rows ``[r*M/R, (r+1)*M/R)`` are stored
    into ``staging_ptrs[r]`` (rank r's staging buffer ``[R, M/R, N]`` bf16) at slot ``rank``."""
    world = len(staging_ptrs)
    m, k = a.shape
    n = b.shape[1]
    assert m % world == 0
    a2, a_mn, lda = cuda_ops._operand(a, 1)  # pylint: disable=protected-access
    b2, b_mn, ldb = cuda_ops._operand(b, 0)  # pylint: disable=protected-access
    fp = FusedParams()
    fp.ag_world = 1
    for r, p in enumerate(staging_ptrs):
        fp.rs_dst[r] = p
    fp.rs_world, fp.rs_rank, fp.rs_rows_per_rank = world, rank, m // world
    cap = max_ctas or (cuda_ops._sm_count(a.device) - cuda_ops.COMM_RESERVED_SMS)  # pylint: disable=protected-access
    rc = _lib().axb_gemm_bf16_fused(a2.data_ptr(), b2.data_ptr(), None, m, n, k, lda, ldb, n, a_mn, b_mn,
                                    cuda_ops.status_word(a.device).data_ptr(), cap, ctypes.addressof(fp),
                                    cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_gemm_bf16_fused(rs)")  # pylint: disable=protected-access


def reduce_slots(staging: torch.Tensor, out: torch.Tensor, *, sumsq_partial: Optional[torch.Tensor] = None) -> None:
    """``out = sum_r staging[r]`` (fp32 accumulation, fixed order, bf16 result)."""
    slots = staging.shape[0]
    n = out.numel()
    assert staging.numel() == slots * n and staging.is_contiguous() and out.is_contiguous()
    rc = _lib().axb_reduce_slots(staging.data_ptr(), out.data_ptr(), slots, n,
                                 None if sumsq_partial is None else sumsq_partial.data_ptr(),
                                 cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_reduce_slots")  # pylint: disable=protected-access


def signal_peers(peer_flag_ptrs_dev: torch.Tensor, world: int, slot: int, value: int) -> None:
    rc = _lib().axb_signal_peers(peer_flag_ptrs_dev.data_ptr(), world, slot, value, cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_signal_peers")  # pylint: disable=protected-access


def wait_flags(flags: torch.Tensor, count: int, value: int) -> None:
    rc = _lib().axb_wait_flags(flags.data_ptr(), count, value, cuda_ops.status_word(flags.device).data_ptr(),
                               cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_wait_flags")  # pylint: disable=protected-access
