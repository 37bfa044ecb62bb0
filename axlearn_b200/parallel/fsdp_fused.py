"""FSDP over NVLink peer memory with the collectives fused into the GEMMs.

Drop-in alternative to ``fsdp.LayerParamGatherer`` for stacked layers whose storage-sharded
leaves live in symmetric (peer-mapped) memory:

* **No gather step.**  ``get(i)`` hands the layer full-shape *views* of per-leaf gather buffers
  (two per leaf, alternating with the layer's parity).  Each weight matrix in them is gathered
  by copy warps that ride inside a GEMM kernel (``ops/fused_comm.py``):

  - in steady state the matrix of layer ``i +/- 1`` is gathered by the GEMM that uses the same
    matrix of layer ``i`` (``gemm_carrying_gather``): the transfer hides under that GEMM, is
    complete by stream order when the next layer starts, and no kernel ever waits on a flag;
  - a matrix that nobody gathered ahead of time (the first layer of a step) is gathered by the
    very GEMM that consumes it (``ag_gemm``): tiles of the rank's own slab are read in place
    while the peers' slabs arrive, later tiles wait on per-slab flags (bounded).

* **No reduce-scatter step.**  The weight-gradient GEMM of a registered matrix stores each
  output row into the owning rank's staging slot (``fused_comm.gemm_rs``); after the layer's
  backward every rank signals its peers, and on the side stream the owner waits for all
  signals (bounded) and reduces its slots in rank order straight into ``stacked.grad[i]``.

Synchronisation across ranks: one barrier per step before the first gather (peers must have
finished their optimizer update), per-layer flags for the gradient partials.  Staging exists
for every layer (full-size bf16 gradients, sharded storage of everything else makes room for
it), so no staging slot is reused within a step.

The reference leaves all of this to XLA's SPMD partitioner and NCCL; see
``axlearn_b200/parallel/fsdp.py`` for the library-collective path with identical semantics,
which stays the oracle in tests.
"""

from __future__ import annotations

import math
import os
from typing import Any, Optional, Sequence

import torch

from axlearn_b200.parallel import fsdp, symm

ENABLED = os.environ.get("AXB200_FUSED_FSDP", "1") != "0"


class PendingMatrix:
    """One 2-D weight matrix of one layer inside a gather buffer."""

    __slots__ = ("full", "shard_ptrs", "state", "rank", "world", "layer", "gathered", "staging_ptrs", "carry")

    def __init__(self, full, shard_ptrs, state, rank, world, layer, gathered, staging_ptrs):
        self.full = full                # [rows, cols] view of the gather buffer
        self.shard_ptrs = shard_ptrs    # address of every rank's row-slab of this layer's matrix
        self.state = state              # _MatrixState of the buffer (flags, cnt, epoch, holds)
        self.rank, self.world = rank, world
        self.layer = layer
        self.gathered = gathered        # the buffer already holds this layer's matrix
        self.staging_ptrs = staging_ptrs  # every rank's staging buffer [R, rows/R, cols]
        # (shard_ptrs, _MatrixState, layer) of the matrix to gather for the neighbouring layer
        # inside this matrix's forward GEMM.
        self.carry = None

    def take_carry(self):
        """The pending neighbour gather, marked as issued (call right before launching it)."""
        c, self.carry = self.carry, None
        if c is None:
            return None
        ptrs, state, layer = c
        state.holds = layer
        return ptrs, state


# Weight matrices whose gather / gradient scatter is fused into the GEMMs, keyed by address.
_pending: dict[int, PendingMatrix] = {}


def lookup(w: torch.Tensor) -> Optional[PendingMatrix]:
    if not _pending:
        return None
    return _pending.get(w.data_ptr())


class _MatrixState:
    def __init__(self, full2d: torch.Tensor, world: int):
        self.full = full2d
        self.flags = torch.zeros(world, dtype=torch.int32, device=full2d.device)
        self.cnt = torch.zeros(world, dtype=torch.int32, device=full2d.device)
        self.epoch = 0
        self.holds = -1  # layer whose matrix the buffer holds (or will, by stream order)


class _Leaf:
    """Geometry of one stacked, storage-sharded leaf: ``[L, batch..., rows/R, cols...]``."""

    def __init__(self, stacked: torch.Tensor, plan: fsdp.LeafPlan, sym: symm.SymmetricBuffer, num_layers: int):
        self.stacked, self.plan, self.sym = stacked, plan, sym
        shape = tuple(stacked.shape[1:])
        d = plan.dim
        self.nb = math.prod(shape[:d])
        self.rows_local = shape[d]
        self.cols = math.prod(shape[d + 1:])
        self.world = plan.world
        self.full_shape = shape[:d] + (self.rows_local * self.world,) + shape[d + 1:]
        dev = stacked.device
        rows = self.rows_local * self.world
        # Two gather buffers: layer i lives in buffer i % 2 while its neighbour arrives in the other.
        self.buffers = [torch.empty(self.full_shape, dtype=stacked.dtype, device=dev) for _ in range(2)]
        self.mats = [
            [_MatrixState(buf.reshape(self.nb, rows, self.cols)[j], self.world) for j in range(self.nb)]
            for buf in self.buffers
        ]
        # Staging for the gradient partials of every layer: [L, nb, R, rows/R, cols].
        self.staging, self.staging_sym = symm.symmetric_empty_like_sharded(
            (num_layers, self.nb, self.world, self.rows_local, self.cols), stacked.dtype, plan.group, dev)

    def shard_ptrs(self, i: int) -> list[list[int]]:
        """Per matrix of layer ``i``: the address of every rank's slab."""
        shard = self.stacked[i]
        peer_base = self.sym.peer_addresses(shard)
        mat_bytes = self.rows_local * self.cols * shard.element_size()
        return [[p + j * mat_bytes for p in peer_base] for j in range(self.nb)]


class FusedLayerGatherer:
    """Same interface as ``fsdp.LayerParamGatherer``; see the module docstring."""

    sharded = True

    def __init__(self, stacked: Any, plans: Any, num_layers: int):
        from axlearn_b200.common.utils import flatten_items

        self._leaves = [t for _, t in flatten_items(stacked)]
        self._plans = [p for _, p in flatten_items(plans, is_leaf=lambda x: isinstance(x, fsdp.LeafPlan))]
        self._num_layers = num_layers
        dev = self._leaves[0].device
        self._device = dev
        self._stream = fsdp.comm_stream(dev)
        self._fused: list[Optional[_Leaf]] = []
        group = None
        for t, p in zip(self._leaves, self._plans):
            if p.world > 1:
                sym = symm.find(t)
                if sym is None:
                    raise ValueError("storage-sharded leaf is not in symmetric memory")
                self._fused.append(_Leaf(t, p, sym, num_layers))
                group = p.group
            else:
                self._fused.append(None)
        self._group = group
        self._world = next(l.world for l in self._fused if l is not None)
        self._rank = next(l.sym.rank for l in self._fused if l is not None)
        # Per-layer flags: flags[i * world + r] = epoch once rank r's partials of layer i landed.
        self._flags, self._flags_sym = symm.symmetric_empty_like_sharded(
            (num_layers * self._world,), torch.int32, group, dev)
        self._flags.zero_()
        self._flag_ptrs = symm.device_pointer_array(self._flags_sym.peer_ptrs, dev)
        # The gatherer is built lazily inside the first step, after that step's `begin_step_all`:
        # start at 1 so that the zero-initialised flags never read as "already signalled".
        self._epoch = 1
        self._current: Optional[int] = None
        self._current_records: list[list[PendingMatrix]] = []
        self._accumulate = False
        self._flags_sym.barrier()

    # ------------------------------------------------------------------ step protocol
    def begin_step(self, accumulate: bool = False) -> None:
        """Cross-rank barrier: peers' parameter shards are final, and their reductions of the
        previous step (or micro-batch) no longer read the staging buffers.  ``accumulate``:
        this micro-batch's gradients are added to what ``stacked.grad`` already holds."""
        self._epoch += 1
        self._accumulate = accumulate
        if not accumulate:
            self.invalidate()
        else:
            # The reductions of the previous micro-batch run on the side stream.
            torch.cuda.current_stream(self._device).wait_stream(self._stream)
        self._flags_sym.barrier()

    def invalidate(self) -> None:
        """Forgets what the gather buffers hold (the shards changed, e.g. after an update)."""
        self._current = None
        for leaf in self._fused:
            if leaf is not None:
                for mats in leaf.mats:
                    for ms in mats:
                        ms.holds = -1

    def get(self, i: int) -> list[torch.Tensor]:
        out = []
        self._current, self._current_records = i, []
        for t, leaf in zip(self._leaves, self._fused):
            if leaf is None:
                out.append(t[i])
                self._current_records.append([])
                continue
            records = []
            for j, (ms, ptrs) in enumerate(zip(leaf.mats[i % 2], leaf.shard_ptrs(i))):
                staging_ptrs = leaf.staging_sym.peer_addresses(leaf.staging[i, j])
                rec = PendingMatrix(ms.full, ptrs, ms, self._rank, self._world, i, ms.holds == i, staging_ptrs)
                _pending[ms.full.data_ptr()] = rec
                records.append(rec)
            self._current_records.append(records)
            out.append(leaf.buffers[i % 2])
        return out

    def prefetch(self, i: int) -> None:
        """Layer ``i`` comes next: let the current layer's GEMMs carry its gathers."""
        cur = self._current
        if cur is None or not 0 <= i < self._num_layers or abs(i - cur) != 1:
            return
        for leaf, records in zip(self._fused, self._current_records):
            if leaf is None:
                continue
            for rec, ms, ptrs in zip(records, leaf.mats[i % 2], leaf.shard_ptrs(i)):
                if ms.holds != i:
                    rec.carry = (ptrs, ms, i)

    def scatter_grads(self, i: int, full_grads: Sequence[Optional[torch.Tensor]]) -> None:
        from axlearn_b200.ops import fused_comm

        # Replicated leaves: accumulate locally (summed over ranks later by sync_grads).
        for t, leaf, g in zip(self._leaves, self._fused, full_grads):
            if leaf is None and g is not None:
                fsdp.accumulate_grad_slice(t, i, g)
            elif leaf is not None and g is not None:
                raise RuntimeError("a fused FSDP leaf received a dense gradient; its weight-gradient GEMM "
                                   "did not go through the fused reduce-scatter path")
        cur = torch.cuda.current_stream(self._device)
        # All of this rank's partials for layer i are queued on `cur`: tell the peers.
        fused_comm.signal_peers(self._flag_ptrs, self._world, slot=i * self._world + self._rank, value=self._epoch)
        self._stream.wait_stream(cur)
        with torch.cuda.stream(self._stream):
            fused_comm.wait_flags(self._flags[i * self._world:(i + 1) * self._world], self._world, self._epoch)
            for t, leaf in zip(self._leaves, self._fused):
                if leaf is None:
                    continue
                if t.grad is None:
                    raise RuntimeError("gradient buffers of stacked leaves must be allocated before backward")
                grad_i = t.grad[i].reshape(leaf.nb, leaf.rows_local * leaf.cols)
                for j in range(leaf.nb):
                    fused_comm.reduce_slots(leaf.staging[i, j], grad_i[j], accumulate=self._accumulate)
                fsdp._touched.setdefault(id(t), set()).add(i)  # pylint: disable=protected-access


_active: list = []


def register(gatherer: "FusedLayerGatherer") -> None:
    _active.append(gatherer)


def reset() -> None:
    """Forgets every registered gatherer (a new trainer in the same process starts clean)."""
    _active.clear()


def begin_step_all(accumulate: bool = False) -> None:
    """Called by the trainer before every forward/backward pass: at the start of a step (after
    the previous optimizer update) and, with ``accumulate``, before each further micro-batch."""
    for g in _active:
        g.begin_step(accumulate)


def invalidate_all() -> None:
    """Called after anything rewrites the parameter shards (optimizer update, restore)."""
    for g in _active:
        g.invalidate()


def make_symmetric(stacked: torch.Tensor, plan: fsdp.LeafPlan) -> torch.Tensor:
    """A copy of ``stacked`` placed in symmetric memory of the leaf's storage group."""
    out, _ = symm.symmetric_empty_like_sharded(tuple(stacked.shape), stacked.dtype, plan.group, stacked.device)
    out.copy_(stacked)
    return out


def supported(leaves: Sequence[torch.Tensor], plans: Sequence[fsdp.LeafPlan]) -> bool:
    """Fused FSDP needs CUDA, a real multi-rank storage group and symmetric shadows."""
    if not ENABLED:
        return False
    any_sharded = False
    for t, p in zip(leaves, plans):
        if p.world > 1:
            any_sharded = True
            if not t.is_cuda or p.world > 8 or symm.find(t) is None or t.dtype != torch.bfloat16:
                return False
            cols = math.prod(t.shape[2 + p.dim:])
            if (t.shape[1 + p.dim] * cols) % 8 or cols % 8:
                return False
    return any_sharded
