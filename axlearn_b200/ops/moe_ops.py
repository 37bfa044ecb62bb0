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
import os
from typing import Optional

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


# ------------------------------------------------------------------------------------------
# Grouped GEMM over expert-sorted, block-padded rows (drop-free mixture of experts).
# ------------------------------------------------------------------------------------------

# Every expert's run of rows starts on a multiple of this.  256 rows is one output tile of the
# CTA-pair GEMM; AXB200_MOE_GROUP_BLOCK=128 keeps the single-CTA kernel's tile (less padding).
GROUP_BLOCK = int(os.environ.get("AXB200_MOE_GROUP_BLOCK", "256"))
if GROUP_BLOCK < 128 or GROUP_BLOCK % 128:
    raise ValueError(f"AXB200_MOE_GROUP_BLOCK must be a multiple of 128, got {GROUP_BLOCK}")


def padded_group_layout(expert_of_pair: torch.Tensor, num_experts: int, max_rows: Optional[int] = None):
    """Sorted, block-padded placement of ``P`` (token, choice) pairs.

    Returns ``(dest [P] int32, offsets [E + 1] int32, block_expert [R / GROUP_BLOCK] int32, R)``:
    pair ``p`` goes to row ``dest[p]`` of an ``[R, M]`` buffer in which expert ``e`` owns rows
    ``[offsets[e], offsets[e + 1])`` (a multiple of ``GROUP_BLOCK`` each, its pairs first -- in pair
    order -- and zero rows after them); ``block_expert`` names the owner of every block of
    ``GROUP_BLOCK`` rows (-1 for the unused tail).  ``R`` is a static bound, so nothing here
    synchronises with the host.

    Pairs whose expert is negative (an expert that lives on another rank) get ``dest = -1``.  With
    ``max_rows`` the buffer is capped at that many rows (rounded up to the block): runs are cut at
    the cap and the pairs beyond it get ``dest = -1`` as well.
    """
    p = expert_of_pair.numel()
    flat = expert_of_pair.reshape(-1).long()
    absent = flat < 0
    flat = torch.where(absent, torch.full_like(flat, num_experts), flat)      # bucket E = "not here"
    counts = torch.bincount(flat, minlength=num_experts + 1)[:num_experts + 1]
    padded = (counts + GROUP_BLOCK - 1) // GROUP_BLOCK * GROUP_BLOCK
    padded[num_experts] = 0
    offsets = torch.zeros(num_experts + 2, dtype=torch.long, device=flat.device)
    offsets[1:] = torch.cumsum(padded, 0)
    rows = (p + num_experts * (GROUP_BLOCK - 1) + GROUP_BLOCK - 1) // GROUP_BLOCK * GROUP_BLOCK
    if max_rows is not None:
        rows = min(rows, (max_rows + GROUP_BLOCK - 1) // GROUP_BLOCK * GROUP_BLOCK)
        offsets = offsets.clamp(max=rows)
    order = torch.argsort(flat, stable=True)
    start_unpadded = torch.cumsum(counts, 0) - counts
    sorted_expert = flat[order]
    rank_in_expert = torch.arange(p, device=flat.device) - start_unpadded[sorted_expert]
    dest_sorted = offsets[:-1][sorted_expert] + rank_in_expert
    dest_sorted = torch.where((sorted_expert < num_experts) & (dest_sorted < offsets[1:][sorted_expert]),
                              dest_sorted, torch.full_like(dest_sorted, -1))
    dest = torch.empty(p, dtype=torch.long, device=flat.device)
    dest[order] = dest_sorted
    offsets = offsets[:num_experts + 1]
    block_start = torch.arange(rows // GROUP_BLOCK, device=flat.device) * GROUP_BLOCK
    block_expert = torch.searchsorted(offsets[1:].contiguous(), block_start, right=True)
    block_expert = torch.where(block_start < offsets[-1], block_expert, torch.full_like(block_expert, -1))
    return dest.to(torch.int32), offsets.to(torch.int32), block_expert.to(torch.int32), rows


def _grouped_argtypes():
    h = _lib()
    if not getattr(h, "_axb_grouped_configured", False):
        h.axb_gemm_bf16_grouped.argtypes = [
            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int,
            c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p]
        h.axb_gemm_bf16_grouped.restype = c_int
        h._axb_grouped_configured = True  # pylint: disable=protected-access
    return h


def _gmm_kernel(x, w, block_expert, transpose_w: bool):
    """``out[r] = x[r] @ (w[g(r)]^T if transpose_w else w[g(r)])`` on the tcgen05 kernel."""
    rows, k = x.shape
    e = w.shape[0]
    n = w.shape[1] if transpose_w else w.shape[2]
    out = torch.zeros((rows, n), dtype=torch.bfloat16, device=x.device)
    rc = _grouped_argtypes().axb_gemm_bf16_grouped(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), rows, n, k, x.stride(0), w.stride(1), out.stride(0),
        0, 0 if transpose_w else 1, 0, 1, e, block_expert.data_ptr(), 0, GROUP_BLOCK,
        cuda_ops.status_word(x.device).data_ptr(), 0, cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_gemm_bf16_grouped")  # pylint: disable=protected-access
    return out


def _tgmm_kernel(x, dy, offsets, num_experts: int):
    """``dw[e] = x[rows of e]^T @ dy[rows of e]`` (bf16 out, fp32 accumulation)."""
    rows, k = x.shape
    n = dy.shape[1]
    dw = torch.empty((num_experts, k, n), dtype=torch.bfloat16, device=x.device)
    rc = _grouped_argtypes().axb_gemm_bf16_grouped(
        x.data_ptr(), dy.data_ptr(), dw.data_ptr(), k, n, rows, x.stride(0), dy.stride(0), n,
        1, 1, 0, 2, num_experts, offsets.data_ptr(), k * n, GROUP_BLOCK,
        cuda_ops.status_word(x.device).data_ptr(), 0, cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_gemm_bf16_grouped")  # pylint: disable=protected-access
    return dw


def _grouped_kernel_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (_use_kernels(x) and w.dtype == torch.bfloat16 and x.shape[0] % GROUP_BLOCK == 0
            and w.shape[1] % 64 == 0 and w.shape[2] % 64 == 0)


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offsets, block_expert):
        x = x.contiguous()
        w = w.contiguous()
        ctx.save_for_backward(x, w, offsets, block_expert)
        return _gmm_kernel(x, w, block_expert, transpose_w=False)

    @staticmethod
    def backward(ctx, g):
        x, w, offsets, block_expert = ctx.saved_tensors
        g = g.contiguous()
        dx = _gmm_kernel(g, w, block_expert, transpose_w=True) if ctx.needs_input_grad[0] else None
        dw = _tgmm_kernel(x, g, offsets, w.shape[0]) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def grouped_linear_reference(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """Per-expert matmuls over the row ranges (synchronises to read the offsets): the oracle of
    the grouped kernel and the path for CPU / non-bf16 inputs."""
    out = x.new_zeros((x.shape[0], w.shape[2]))
    bounds = offsets.tolist()
    pieces = []
    for e in range(w.shape[0]):
        lo, hi = bounds[e], bounds[e + 1]
        pieces.append(x[lo:hi] @ w[e].to(x.dtype))
    used = torch.cat(pieces, dim=0) if pieces else out[:0]
    return torch.cat([used, out[used.shape[0]:]], dim=0)


def grouped_linear(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor,
                   block_expert: torch.Tensor) -> torch.Tensor:
    """``x [R, K]`` (rows laid out by ``padded_group_layout``) times ``w [E, K, N]`` -> ``[R, N]``:
    the reference's ``gmm(lhs, rhs, group_sizes)`` (axlearn/common/megablock/ops.py:15-105) with
    its transposed / per-group-transposed variants as the backward pass."""
    if _grouped_kernel_ok(x, w):
        return _GroupedLinear.apply(x, w, offsets, block_expert)
    return grouped_linear_reference(x, w, offsets)


# ------------------------------------------------------------------------------------------
# Expert-parallel exchange over peer memory: dispatch pushes rows into the owners' memory,
# combine pulls rows out of it (the all-to-all pair fused into the token gather / weighted sum).
# ------------------------------------------------------------------------------------------

_IN_READY, _IN_FREE, _OUT_READY, _OUT_FREE = range(4)


def _peer_argtypes():
    h = _lib()
    if not getattr(h, "_axb_peer_moe_configured", False):
        h.axb_moe_push_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int64, c_int, c_void_p]
        h.axb_moe_pull_combine.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                           c_int64, c_int, c_int, c_void_p]
        h.axb_moe_pull_row_dots.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                            c_int64, c_int, c_int, c_void_p]
        for f in (h.axb_moe_push_rows, h.axb_moe_pull_combine, h.axb_moe_pull_row_dots):
            f.restype = c_int
        h._axb_peer_moe_configured = True  # pylint: disable=protected-access
    return h


class ExpertExchange:
    """Symmetric in/out boxes ``[E_local, world, slots, M]`` (bf16) of one expert-parallel group
    plus the four flag sets of the hand-shake:

    * push: wait until the owners have emptied their in-boxes of my previous rows (``IN_FREE``),
      store my rows into the owners' in-boxes, raise ``IN_READY`` there, wait for everybody's
      ``IN_READY`` here, copy the in-box out, raise ``IN_FREE`` at the senders;
    * pull: wait until everybody has read my previous out-box (``OUT_FREE``), fill it, raise
      ``OUT_READY`` at the readers, wait for the owners' ``OUT_READY``, read rows out of the
      owners' out-boxes, raise ``OUT_FREE`` at the owners.

    Every wait is a bounded device-side wait that reports through the status word.  All ranks
    must issue the same sequence of pushes and pulls (true for SPMD training steps).  With
    ``group=None`` the "group" is this GPU alone (the kernels and the protocol still run: used by
    single-GPU tests)."""

    def __init__(self, experts_per_rank: int, slots: int, model_dim: int, group, device: torch.device):
        from axlearn_b200.parallel import symm

        self.experts_per_rank, self.slots, self.model_dim = experts_per_rank, slots, model_dim
        if group is None:
            self.world, self.rank = 1, 0
            shape = (experts_per_rank, 1, slots, model_dim)
            self.inbox = torch.empty(shape, dtype=torch.bfloat16, device=device)
            self.outbox = torch.empty(shape, dtype=torch.bfloat16, device=device)
            self.flags = torch.zeros(4, dtype=torch.int32, device=device)
            in_ptrs, out_ptrs, flag_ptrs = [self.inbox.data_ptr()], [self.outbox.data_ptr()], [self.flags.data_ptr()]
        else:
            import torch.distributed as dist

            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            shape = (experts_per_rank, self.world, slots, model_dim)
            self.inbox, in_sym = symm.symmetric_empty_like_sharded(shape, torch.bfloat16, group, device)
            self.outbox, out_sym = symm.symmetric_empty_like_sharded(shape, torch.bfloat16, group, device)
            self.flags, flag_sym = symm.symmetric_empty_like_sharded((4 * self.world,), torch.int32, group, device)
            self.flags.zero_()
            torch.cuda.synchronize(device)
            flag_sym.barrier()
            in_ptrs, out_ptrs, flag_ptrs = in_sym.peer_ptrs, out_sym.peer_ptrs, flag_sym.peer_ptrs
            self._keep = (in_sym, out_sym, flag_sym)
        arr = ctypes.c_void_p * self.world
        self._in_bases, self._out_bases = arr(*in_ptrs), arr(*out_ptrs)
        self._flag_ptrs = symm.device_pointer_array(flag_ptrs, device)
        self._push_epoch = 0
        self._pull_epoch = 0

    # -------------------------------------------------------------- hand-shake helpers
    def _signal(self, kind: int, value: int) -> None:
        from axlearn_b200.ops import fused_comm

        fused_comm.signal_peers(self._flag_ptrs, self.world, kind * self.world + self.rank, value)

    def _wait(self, kind: int, value: int) -> None:
        from axlearn_b200.ops import fused_comm

        fused_comm.wait_flags(self.flags[kind * self.world:(kind + 1) * self.world], self.world, value)

    # -------------------------------------------------------------- push
    def push(self, src: torch.Tensor, row_source: torch.Tensor, scale) -> torch.Tensor:
        """``src [T, M]``; ``row_source [E * slots]`` = the row of ``src`` that fills each flat
        (expert, slot) row, -1 for an empty slot (filled with zeros); optional per-row scale.
        Returns this rank's experts' input ``[E_local, world * slots, M]``."""
        self._push_epoch += 1
        p = self._push_epoch
        if p > 1:
            self._wait(_IN_FREE, p - 1)
        rows = self.world * self.experts_per_rank * self.slots
        assert row_source.numel() == rows and src.shape[1] == self.model_dim
        rc = _peer_argtypes().axb_moe_push_rows(
            src.data_ptr(), row_source.data_ptr(), None if scale is None else scale.data_ptr(), self._in_bases,
            self.world, self.rank, self.slots, self.experts_per_rank, rows, self.model_dim,
            cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_moe_push_rows")  # pylint: disable=protected-access
        self._signal(_IN_READY, p)
        self._wait(_IN_READY, p)
        out = self.inbox.clone().reshape(self.experts_per_rank, self.world * self.slots, self.model_dim)
        self._signal(_IN_FREE, p)
        return out

    # -------------------------------------------------------------- pull
    def _pull_begin(self, y: torch.Tensor) -> None:
        self._pull_epoch += 1
        q = self._pull_epoch
        if q > 1:
            self._wait(_OUT_FREE, q - 1)
        self.outbox.copy_(y.reshape(self.outbox.shape))
        # The copy is an ordinary kernel / copy engine write to local memory: the release store
        # of the flag kernel (after a system fence) orders it before the flag.
        self._signal(_OUT_READY, q)
        self._wait(_OUT_READY, q)

    def _pull_end(self) -> None:
        self._signal(_OUT_FREE, self._pull_epoch)

    def pull_combine(self, y: torch.Tensor, dest: torch.Tensor, weight) -> torch.Tensor:
        """``y [E_local, world * slots, M]`` (this rank's experts' outputs) ->
        ``out[t] = sum_k weight[t, k] * row dest[t, k]`` of the owners' outputs."""
        self._pull_begin(y)
        tokens, k = dest.shape
        out = torch.empty((tokens, self.model_dim), dtype=torch.bfloat16, device=y.device)
        rc = _peer_argtypes().axb_moe_pull_combine(
            self._out_bases, self.world, self.rank, self.slots, self.experts_per_rank, dest.data_ptr(),
            None if weight is None else weight.data_ptr(), out.data_ptr(), tokens, k, self.model_dim,
            cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_moe_pull_combine")  # pylint: disable=protected-access
        self._pull_end()
        return out

    def pull_row_dots(self, a: torch.Tensor, y: torch.Tensor, dest: torch.Tensor) -> torch.Tensor:
        """``out[t, k] = <a[t], row dest[t, k] of the owners' y>`` (gradient of the gate weights)."""
        self._pull_begin(y)
        tokens, k = dest.shape
        out = torch.empty((tokens, k), dtype=torch.float32, device=a.device)
        rc = _peer_argtypes().axb_moe_pull_row_dots(
            a.data_ptr(), self._out_bases, self.world, self.rank, self.slots, self.experts_per_rank,
            dest.data_ptr(), out.data_ptr(), tokens, k, self.model_dim, cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_moe_pull_row_dots")  # pylint: disable=protected-access
        self._pull_end()
        return out


_exchanges: dict[tuple, ExpertExchange] = {}


def expert_exchange(experts_per_rank: int, slots: int, model_dim: int, group, device) -> ExpertExchange:
    key = (experts_per_rank, slots, model_dim, None if group is None else id(group), str(device))
    if key not in _exchanges:
        _exchanges[key] = ExpertExchange(experts_per_rank, slots, model_dim, group, device)
    return _exchanges[key]


class _EpDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dest, inv, ex):
        k = dest.shape[1]
        row_source = torch.where(inv >= 0, inv // k, inv).contiguous()
        ctx.save_for_backward(dest)
        ctx.ex = ex
        return ex.push(x.contiguous(), row_source, None)

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        return ctx.ex.pull_combine(g.contiguous(), dest, None), None, None, None


class _EpCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, weight, dest, inv, ex):
        y = y.contiguous()
        weight = weight.float().contiguous()
        ctx.save_for_backward(y, weight, dest, inv)
        ctx.ex = ex
        return ex.pull_combine(y, dest, weight)

    @staticmethod
    def backward(ctx, g):
        y, weight, dest, inv = ctx.saved_tensors
        ex = ctx.ex
        g = g.contiguous()
        k = dest.shape[1]
        dw = ex.pull_row_dots(g, y, dest)
        row_source = torch.where(inv >= 0, inv // k, inv).contiguous()
        w_of_row = weight.reshape(-1)[inv.clamp(min=0).long()].contiguous()
        dy = ex.push(g, row_source, w_of_row)
        return dy, dw, None, None, None


def peer_exchange_ok(x: torch.Tensor) -> bool:
    return _use_kernels(x) and os.environ.get("AXB_MOE_PEER_EXCHANGE", "1") != "0"


def ep_dispatch(x: torch.Tensor, dest: torch.Tensor, ex: ExpertExchange) -> torch.Tensor:
    """``x [T, M]``, ``dest [T, K]`` (expert-major flat rows ``e * slots + slot``, -1 = dropped)
    -> this rank's experts' inputs ``[E_local, world * slots, M]``."""
    dest = dest.to(torch.int32).contiguous()
    rows = ex.world * ex.experts_per_rank * ex.slots
    return _EpDispatch.apply(x, dest, inverse_pairs(dest, rows), ex)


def ep_combine(y: torch.Tensor, weight: torch.Tensor, dest: torch.Tensor, ex: ExpertExchange) -> torch.Tensor:
    """``y [E_local, world * slots, M]`` -> ``[T, M]`` (weighted sum over each token's choices)."""
    dest = dest.to(torch.int32).contiguous()
    rows = ex.world * ex.experts_per_rank * ex.slots
    return _EpCombine.apply(y, weight, dest, inverse_pairs(dest, rows), ex)


# ------------------------------------------------------------------------------------------
# Routing (csrc/moe_gate.cu): scores, top-k, capacity positions and aux-loss sums.
# ------------------------------------------------------------------------------------------

_gate_configured = False


def _gate_lib():
    global _gate_configured
    h = cuda_ops.lib()
    if not _gate_configured:
        c_float = ctypes.c_float
        h.axb_moe_gate_parts.argtypes = [c_int]
        h.axb_moe_gate_parts.restype = c_int
        h.axb_moe_gate_fwd.argtypes = [c_void_p] * 8 + [c_int] * 5 + [c_float, c_int, c_void_p]
        h.axb_moe_gate_fwd.restype = c_int
        h.axb_moe_gate_bwd.argtypes = [c_void_p] * 7 + [c_int] * 4 + [c_float, c_int, c_void_p]
        h.axb_moe_gate_bwd.restype = c_int
        _gate_configured = True
    return h


def gate_kernel_ok(logits: torch.Tensor, k: int) -> bool:
    from axlearn_b200.ops import dispatch as op_dispatch

    return (logits.is_cuda and logits.shape[-1] <= 256 and 1 <= k <= min(8, logits.shape[-1])
            and not op_dispatch._flags.force_reference)  # pylint: disable=protected-access


def topk_gate_reference(logits: torch.Tensor, k: int, capacity: int, logit_cap: float = 0.0, sigmoid: bool = False):
    """The same routing in PyTorch statements (oracle; ``logits [G, S, E]``)."""
    g, s, e = logits.shape
    x = logits.float()
    if logit_cap > 0:
        x = logit_cap * torch.tanh(x / logit_cap)
    lse = torch.logsumexp(x, dim=-1)
    score = torch.sigmoid(x) if sigmoid else torch.softmax(x, dim=-1)
    gate, index = score.topk(k, dim=-1)
    flat = index.permute(0, 2, 1).reshape(g, k * s)                      # choice-major priority
    keys = (torch.arange(g, device=x.device)[:, None] * e + flat).reshape(-1)
    order = torch.sort(keys, stable=True).indices
    cnt = torch.bincount(keys, minlength=g * e)
    starts = cnt.cumsum(0) - cnt
    pos = torch.empty_like(keys)
    pos[order] = torch.arange(keys.numel(), device=x.device) - starts[keys[order]]
    slot = torch.where(pos < capacity, pos, torch.full_like(pos, -1)).reshape(g, k, s).permute(0, 2, 1).contiguous()
    counts = torch.stack([torch.nn.functional.one_hot(index[..., j], e).sum(dim=1) for j in range(k)], dim=1)
    return index, gate, slot, counts, score.sum(dim=1), lse


class _TopkGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, capacity, logit_cap, sigmoid):
        g, s, e = logits.shape
        dev = logits.device
        logits = logits.contiguous()
        h = _gate_lib()
        index = torch.empty((g, s, k), dtype=torch.int32, device=dev)
        gate = torch.empty((g, s, k), dtype=torch.float32, device=dev)
        slot = torch.empty((g, s, k), dtype=torch.int32, device=dev)
        counts = torch.empty((g, k, e), dtype=torch.int32, device=dev)
        proxy = torch.empty((g, e), dtype=torch.float32, device=dev)
        lse = torch.empty((g, s), dtype=torch.float32, device=dev)
        part = torch.empty((g, h.axb_moe_gate_parts(s), e), dtype=torch.float32, device=dev)
        rc = h.axb_moe_gate_fwd(logits.data_ptr(), index.data_ptr(), gate.data_ptr(), slot.data_ptr(),
                                counts.data_ptr(), proxy.data_ptr(), lse.data_ptr(), part.data_ptr(), g, s, e, k,
                                int(capacity), float(logit_cap), 1 if sigmoid else 0, cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_moe_gate_fwd")  # pylint: disable=protected-access
        cuda_ops.launch_count += 1
        ctx.save_for_backward(logits, index, lse)
        ctx.args = (k, float(logit_cap), bool(sigmoid))
        index64, slot64, counts64 = index.long(), slot.long(), counts.long()
        ctx.mark_non_differentiable(index64, slot64, counts64)
        return index64, gate, slot64, counts64, proxy, lse

    @staticmethod
    def backward(ctx, _di, d_gate, _ds, _dc, d_proxy, d_lse):
        logits, index, lse = ctx.saved_tensors
        k, cap, sigmoid = ctx.args
        g, s, e = logits.shape
        d_logits = torch.empty_like(logits)
        opt = lambda t: None if t is None else t.float().contiguous()
        d_gate, d_proxy, d_lse = opt(d_gate), opt(d_proxy), opt(d_lse)
        if d_gate is None:
            d_gate = torch.zeros((g, s, k), dtype=torch.float32, device=logits.device)
        rc = _gate_lib().axb_moe_gate_bwd(
            logits.data_ptr(), index.data_ptr(), lse.data_ptr(), d_gate.data_ptr(), cuda_ops._p(d_proxy),  # pylint: disable=protected-access
            cuda_ops._p(d_lse), d_logits.data_ptr(), g, s, e, k, cap, 1 if sigmoid else 0, cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_moe_gate_bwd")  # pylint: disable=protected-access
        return d_logits, None, None, None, None


def topk_gate(logits: torch.Tensor, k: int, capacity: int, *, logit_cap: float = 0.0, sigmoid: bool = False):
    """Routing of ``logits [G, S, E]`` (fp32): ``(index [G,S,K], gate [G,S,K], slot [G,S,K],
    counts [G,K,E], score_sums [G,E], lse [G,S])``.  ``gate`` are the chosen experts' scores,
    ``slot`` the capacity positions in choice-major priority order (-1 = dropped), ``counts`` the
    tokens per (choice, expert), ``score_sums`` the per-expert sums of the scores over the group's
    tokens and ``lse`` the per-token log-sum-exp of the (capped) logits; ``gate``, ``score_sums`` and
    ``lse`` are differentiable."""
    if gate_kernel_ok(logits, k):
        return _TopkGate.apply(logits.float(), int(k), int(capacity), float(logit_cap), bool(sigmoid))
    return topk_gate_reference(logits, k, capacity, logit_cap, sigmoid)
