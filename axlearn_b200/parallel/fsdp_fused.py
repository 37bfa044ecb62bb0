"""FSDP over NVLink peer memory with the collectives fused into the GEMMs.

Drop-in alternative to ``fsdp.LayerParamGatherer`` for stacked layers whose storage-sharded
leaves live in symmetric (peer-mapped) memory:

* **No gather step.**  ``get(i)`` hands the layer full-shape *views* of per-leaf scratch buffers
  that are still empty, and registers each weight matrix in them as a pending gather.  The first
  ``linear`` that consumes a matrix runs ``fused_comm.ag_gemm``: copy CTAs of the GEMM kernel
  pull the peers' row-slabs into the buffer while the other CTAs start on the local slab.  Later
  users of the same matrix in that layer (the data-gradient GEMM) find it complete.
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
COPY_CTAS = int(os.environ.get("AXB200_AG_COPY_CTAS", "8"))


class PendingMatrix:
    """One 2-D weight matrix inside a gather buffer."""

    __slots__ = ("full", "shard_ptrs", "state", "rank", "world", "gathered", "staging_ptrs", "rows", "cols")

    def __init__(self, full, shard_ptrs, state, rank, world, staging_ptrs):
        self.full = full                # [rows, cols] view of the gather buffer
        self.shard_ptrs = shard_ptrs    # address of every rank's row-slab
        self.state = state              # fused_comm.GatherState-like (flags, cnt, epoch)
        self.rank, self.world = rank, world
        self.gathered = False
        self.staging_ptrs = staging_ptrs  # every rank's staging buffer [R, rows/R, cols]
        self.rows, self.cols = full.shape


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
        self.buffer = torch.empty(self.full_shape, dtype=stacked.dtype, device=dev)
        rows = self.rows_local * self.world
        self.mats = [
            _MatrixState(self.buffer.reshape(self.nb, rows, self.cols)[j], self.world) for j in range(self.nb)
        ]
        # Staging for the gradient partials of every layer: [L, nb, R, rows/R, cols].
        self.staging, self.staging_sym = symm.symmetric_empty_like_sharded(
            (num_layers, self.nb, self.world, self.rows_local, self.cols), stacked.dtype, plan.group, dev)


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
        # No SMs are set aside here: the copy CTAs are part of the GEMM launch itself, and the
        # small reduction kernels fit beside resident GEMM CTAs.
        self._flags_sym.barrier()

    # ------------------------------------------------------------------ step protocol
    def begin_step(self) -> None:
        """Cross-rank barrier: peers' parameter shards are final, and their reductions of the
        previous step no longer read the staging buffers."""
        self._epoch += 1
        self._flags_sym.barrier()

    def prefetch(self, i: int) -> None:
        del i  # Gathers are fused into the consuming GEMMs.

    def get(self, i: int) -> list[torch.Tensor]:
        out = []
        for t, leaf in zip(self._leaves, self._fused):
            if leaf is None:
                out.append(t[i])
                continue
            shard = t[i]  # [batch..., rows/R, cols...]
            peer_base = leaf.sym.peer_addresses(shard)
            mat_bytes = leaf.rows_local * leaf.cols * shard.element_size()
            for j, ms in enumerate(leaf.mats):
                shard_ptrs = [p + j * mat_bytes for p in peer_base]
                staging_local = leaf.staging[i, j]
                staging_ptrs = leaf.staging_sym.peer_addresses(staging_local)
                _pending[ms.full.data_ptr()] = PendingMatrix(
                    ms.full, shard_ptrs, ms, self._rank, self._world, staging_ptrs)
            out.append(leaf.buffer)
        return out

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
                    fused_comm.reduce_slots(leaf.staging[i, j], grad_i[j])
                fsdp._touched.setdefault(id(t), set()).add(i)  # pylint: disable=protected-access


_active: list = []


def register(gatherer: "FusedLayerGatherer") -> None:
    _active.append(gatherer)


def begin_step_all() -> None:
    """Called by the trainer at the start of every step (after the previous optimizer update)."""
    for g in _active:
        g.begin_step()


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
