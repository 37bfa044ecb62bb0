"""Fused compute+collective ops over NVLink peer memory.

* ``ag_gemm``: ``x @ W`` where ``W`` is stored as one contiguous row-slab per rank (FSDP).  One
  extra warp in every CTA of the GEMM kernel pulls its share of the peers' slabs into a local
  full-size buffer with bulk asynchronous copies while the GEMM starts on the rank's own slab
  (read in place); tiles that need a remote slab wait on a per-slab flag (bounded).  This is the
  reference's "all-gather the bf16 parameters, then matmul" (axlearn/common/attention.py:3803-3850
  shardings, collectives inserted by XLA) as one kernel.
* ``gemm_carrying_gather``: a GEMM on complete operands whose copy warps gather a *different*
  weight (the next layer's) for a later launch, so that in steady state no GEMM ever waits.
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


class GatherJob(ctypes.Structure):
    """Host mirror of ``axb::GatherJob`` (csrc/gemm.cu)."""

    _fields_ = [
        ("src", c_void_p * MAX_PEERS),
        ("dst", c_void_p),
        ("flags", c_void_p),
        ("cnt", c_void_p),
        ("shard_bytes", c_int64),
        ("world", c_int),
        ("rank", c_int),
        ("epoch", c_int),
        ("reserved", c_int),
    ]


class FusedParams(ctypes.Structure):
    """Host mirror of ``axb::FusedParams`` (csrc/gemm.cu)."""

    _fields_ = [
        ("ag", GatherJob * 2),
        ("ag_consume", c_int),
        ("ag_along_k", c_int),
        ("ag_shard_extent", c_int),
        ("reserved", c_int),
        ("rs_dst", c_void_p * MAX_PEERS),
        ("rs_world", c_int),
        ("rs_rank", c_int),
        ("rs_rows_per_rank", c_int),
        ("rs_mode", c_int),
        ("rs_site", c_int),
        ("reserved2", c_int),
        ("rs_counter", c_void_p),
        ("rs_epoch_ptr", c_void_p),
        ("rs_flags", c_void_p * MAX_PEERS),
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
        h.axb_reduce_slots.argtypes = [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p]
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


def _fill_gather(job: GatherJob, shard_ptrs: Sequence[int], state, rank: int) -> None:
    world = len(shard_ptrs)
    rows, cols = state.full.shape
    assert rows % world == 0 and 1 < world <= MAX_PEERS
    state.epoch += 1
    for r, p in enumerate(shard_ptrs):
        job.src[r] = p
    job.dst = state.full.data_ptr()
    job.flags = state.flags.data_ptr()
    job.cnt = state.cnt.data_ptr()
    job.shard_bytes = (rows // world) * cols * 2
    job.world, job.rank, job.epoch = world, rank, state.epoch


def ag_gemm(x: torch.Tensor, *, shard_ptrs: Sequence[int], state: GatherState, rank: int,
            weight_is_nk: bool = False, carry: Optional[tuple] = None, out: Optional[torch.Tensor] = None,
            max_ctas: int = 0) -> torch.Tensor:
    """``x[M, K] @ W`` with W gathered inside the kernel that consumes it.

    ``shard_ptrs[r]`` is the address of rank r's slab (``W[r*rows/R:(r+1)*rows/R]``), its own for
    ``r == rank``.  ``state.full`` has W's full shape: ``[K, N]`` (slabs split the contraction
    dim) or, with ``weight_is_nk``, ``[N, K]`` used as ``x @ W^T`` (slabs split the output dim).
    Tiles inside the rank's own slab are read from the shard itself; the rest wait for the
    slabs as they land.  After the call ``state.full`` holds the whole of W.  ``carry`` =
    ``(shard_ptrs, state)`` of a second, unrelated matrix to gather in the same launch (see
    ``gemm_carrying_gather``).
    """
    full = state.full
    rows, cols = full.shape
    x2 = x.reshape(-1, x.shape[-1])
    m, k = x2.shape
    n = rows if weight_is_nk else cols
    assert (cols if weight_is_nk else rows) == k, (full.shape, x2.shape)
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    fp = FusedParams()
    _fill_gather(fp.ag[0], shard_ptrs, state, rank)
    fp.ag_consume, fp.ag_along_k, fp.ag_shard_extent = 1, 0 if weight_is_nk else 1, rows // len(shard_ptrs)
    if carry is not None:
        _fill_gather(fp.ag[1], carry[0], carry[1], rank)
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


def gemm_carrying_gather(x: torch.Tensor, w: torch.Tensor, *, shard_ptrs: Sequence[int], state: GatherState,
                         rank: int, out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    """``x[M, K] @ w[K, N]`` (``w`` complete and local) while the same kernel's copy warps gather
    *another* matrix -- ``shard_ptrs`` into ``state.full`` -- for a later launch.

    Nothing in this kernel waits for the copy: it hides under the GEMM and is complete, by
    stream order, when the kernel ends (this is how layer i+1's weights arrive during layer i).
    """
    x2 = x.reshape(-1, x.shape[-1])
    m, k = x2.shape
    n = w.shape[1]
    assert w.shape[0] == k
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    fp = FusedParams()
    _fill_gather(fp.ag[0], shard_ptrs, state, rank)
    fp.rs_world = 1
    x2c, a_mn, lda = cuda_ops._operand(x2, 1)  # pylint: disable=protected-access
    w2, b_mn, ldb = cuda_ops._operand(w, 0)  # pylint: disable=protected-access
    cap = max_ctas or (cuda_ops._sm_count(x.device) - cuda_ops.COMM_RESERVED_SMS)  # pylint: disable=protected-access
    rc = _lib().axb_gemm_bf16_fused(x2c.data_ptr(), w2.data_ptr(), out.data_ptr(), m, n, k, lda, ldb,
                                    out.stride(0), a_mn, b_mn, cuda_ops.status_word(x.device).data_ptr(), cap,
                                    ctypes.addressof(fp), cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_gemm_bf16_fused(carry)")  # pylint: disable=protected-access
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
    for r, p in enumerate(staging_ptrs):
        fp.rs_dst[r] = p
    fp.rs_world, fp.rs_rank, fp.rs_rows_per_rank = world, rank, m // world
    cap = max_ctas or (cuda_ops._sm_count(a.device) - cuda_ops.COMM_RESERVED_SMS)  # pylint: disable=protected-access
    rc = _lib().axb_gemm_bf16_fused(a2.data_ptr(), b2.data_ptr(), None, m, n, k, lda, ldb, n, a_mn, b_mn,
                                    cuda_ops.status_word(a.device).data_ptr(), cap, ctypes.addressof(fp),
                                    cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_gemm_bf16_fused(rs)")  # pylint: disable=protected-access


def gemm_allreduce_push(a: torch.Tensor, b: torch.Tensor, *, staging_ptrs: Sequence[int], flag_ptrs: Sequence[int],
                        counter: torch.Tensor, epoch: torch.Tensor, rank: int, site: int, max_ctas: int = 0) -> None:
    """``a[M, K] @ b[K, N]`` whose epilogue is the first half of a small-message all-reduce: every
    row is stored into slot ``rank`` of every peer's staging buffer ``[R, M, N]``
    (``staging_ptrs[r]``), and the last CTA raises flag ``[site * R + rank]`` (= the value in
    ``epoch``, device memory) in every peer's flag array (``flag_ptrs[r]``).  The sum is taken by
    ``OneShotAllReduce.finish`` on every rank."""
    world = len(staging_ptrs)
    m, k = a.shape
    n = b.shape[1]
    assert n % 32 == 0
    a2, a_mn, lda = cuda_ops._operand(a, 1)  # pylint: disable=protected-access
    b2, b_mn, ldb = cuda_ops._operand(b, 0)  # pylint: disable=protected-access
    fp = FusedParams()
    for r in range(world):
        fp.rs_dst[r] = staging_ptrs[r]
        fp.rs_flags[r] = flag_ptrs[r]
    fp.rs_world, fp.rs_rank, fp.rs_rows_per_rank, fp.rs_mode, fp.rs_site = world, rank, m, 1, site
    fp.rs_counter = counter.data_ptr()
    fp.rs_epoch_ptr = epoch.data_ptr()
    cap = max_ctas or (cuda_ops._sm_count(a.device) - cuda_ops.COMM_RESERVED_SMS)  # pylint: disable=protected-access
    rc = _lib().axb_gemm_bf16_fused(a2.data_ptr(), b2.data_ptr(), None, m, n, k, lda, ldb, n, a_mn, b_mn,
                                    cuda_ops.status_word(a.device).data_ptr(), cap, ctypes.addressof(fp),
                                    cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_gemm_bf16_fused(allreduce push)")  # pylint: disable=protected-access


def reduce_slots(staging: torch.Tensor, out: torch.Tensor, *, sumsq_partial: Optional[torch.Tensor] = None,
                 accumulate: bool = False) -> None:
    """``out (+)= sum_r staging[r]`` (fp32 accumulation, fixed order, bf16 result)."""
    slots = staging.shape[0]
    n = out.numel()
    assert staging.numel() == slots * n and staging.is_contiguous() and out.is_contiguous()
    rc = _lib().axb_reduce_slots(staging.data_ptr(), out.data_ptr(), slots, n,
                                 None if sumsq_partial is None else sumsq_partial.data_ptr(),
                                 1 if accumulate else 0, cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_reduce_slots")  # pylint: disable=protected-access


def signal_peers(peer_flag_ptrs_dev: torch.Tensor, world: int, slot: int, value: int) -> None:
    rc = _lib().axb_signal_peers(peer_flag_ptrs_dev.data_ptr(), world, slot, value, cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_signal_peers")  # pylint: disable=protected-access


def wait_flags(flags: torch.Tensor, count: int, value: int) -> None:
    rc = _lib().axb_wait_flags(flags.data_ptr(), count, value, cuda_ops.status_word(flags.device).data_ptr(),
                               cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_wait_flags")  # pylint: disable=protected-access
