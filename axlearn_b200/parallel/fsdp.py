"""Per-layer parameter gathering and gradient scattering for stacked, storage-sharded layers.

A repeated layer stack keeps each parameter as one tensor ``[L, ...local shard...]``.  To run
layer ``i`` every rank needs the full (compute-shape) parameters of that layer; after the
layer's backward each rank keeps only its shard of the gradient.  ``LayerParamGatherer``
does both on a side stream so that the transfer of layer ``i±1`` overlaps the math of layer
``i`` — the job XLA's latency-hiding scheduler does for the reference's scanned layers
(axlearn/common/repeat.py:172-223 with the all-gathers inserted per
axlearn/common/attention.py:3803-3850).

This file is the library-collective implementation (one NCCL/gloo call per parameter); it is
the correctness oracle and the fallback of the fused peer-memory path.
"""

from __future__ import annotations

import os
from typing import Any, Optional, Sequence

import torch
import torch.distributed as dist

from axlearn_b200.parallel import collectives as coll
from axlearn_b200.parallel.mesh import Mesh, current_mesh


# SMs reserved for communication kernels while a sharded layer stack runs (see
# cuda_ops.reserve_sms_for_comm); the launcher caps the library collectives to the same number.
COMM_SMS = int(os.environ.get("AXB200_COMM_SMS", "16"))


class _CommStream:
    """One side stream per device for parameter traffic."""

    _streams: dict = {}

    @classmethod
    def get(cls, device: torch.device):
        if device.type != "cuda":
            return None
        key = device.index if device.index is not None else torch.cuda.current_device()
        if key not in cls._streams:
            cls._streams[key] = torch.cuda.Stream(device=device)
        return cls._streams[key]


def comm_stream(device: torch.device):
    return _CommStream.get(device)


def wait_pending(device: Optional[torch.device] = None) -> None:
    """Makes the current stream wait for all parameter/gradient traffic issued so far."""
    if device is None:
        if not torch.cuda.is_available():
            return
        device = torch.device("cuda", torch.cuda.current_device())
    s = _CommStream.get(device)
    if s is not None:
        torch.cuda.current_stream(device).wait_stream(s)


class LeafPlan:
    """How one stacked leaf is sharded: the storage axes and the (per-layer) dim they split."""

    def __init__(self, mesh: Optional[Mesh], layer_mesh_axes: Optional[Sequence[Any]]):
        self.dim = None
        self.axes: tuple[str, ...] = ()
        self.group = None
        self.world = 1
        if mesh is None or layer_mesh_axes is None:
            return
        for d, entry in enumerate(layer_mesh_axes):
            axes = coll.storage_axes(entry, mesh)
            if axes:
                if self.dim is not None:
                    raise NotImplementedError("a parameter may be storage-sharded on one dim only")
                self.dim, self.axes = d, axes
                self.world = mesh.axis_size(axes)
                self.group = mesh.group(axes)


def gather_leaf(shard: torch.Tensor, plan: LeafPlan) -> torch.Tensor:
    """Full tensor from this rank's ``shard`` (layer slice, no leading L dim)."""
    if plan.world == 1:
        return shard
    return coll.all_gather_raw(shard, plan.group, plan.world, plan.dim)


def scatter_grad_leaf(full_grad: torch.Tensor, plan: LeafPlan) -> torch.Tensor:
    if plan.world == 1:
        return full_grad
    return coll.reduce_scatter_raw(full_grad, plan.group, plan.world, plan.dim)


_touched: dict[int, set] = {}


def reset_grad_slices(stacked: torch.Tensor) -> None:
    """Forgets which layer slices of ``stacked.grad`` were written (call at zero_grad)."""
    _touched.pop(id(stacked), None)


def accumulate_grad_slice(stacked: torch.Tensor, i: int, g: torch.Tensor) -> None:
    """``stacked.grad[i] (+)= g``: the first write after a reset stores, later ones add."""
    if stacked.grad is None:
        stacked.grad = torch.empty_like(stacked)
        _touched[id(stacked)] = set()
    seen = _touched.setdefault(id(stacked), set())
    if i in seen:
        stacked.grad[i].add_(g.to(stacked.grad.dtype))
    else:
        stacked.grad[i].copy_(g)
        seen.add(i)


def finalize_grad_slices(stacked: torch.Tensor, num_layers: int) -> None:
    """Zero-fills slices that received no gradient (layers that did not run)."""
    if stacked.grad is None:
        return
    seen = _touched.get(id(stacked), set())
    for i in range(num_layers):
        if i not in seen:
            stacked.grad[i].zero_()


class LayerParamGatherer:
    """Gathers layer ``i`` of a tree of stacked shards, with one-layer look-ahead."""

    def __init__(self, stacked: Any, plans: Any, num_layers: int):
        from axlearn_b200.common.utils import flatten_items

        self._leaves = [t for _, t in flatten_items(stacked)]
        self._plans = [p for _, p in flatten_items(plans, is_leaf=lambda x: isinstance(x, LeafPlan))]
        self._num_layers = num_layers
        self._ready: dict[int, tuple[list[torch.Tensor], Any]] = {}
        self.sharded = any(p.world > 1 for p in self._plans)
        dev = self._leaves[0].device if self._leaves else torch.device("cpu")
        self._stream = comm_stream(dev) if self.sharded else None
        self._device = dev
        if self.sharded and dev.type == "cuda":
            # Collectives run beside compute: keep a few SMs free for them.
            from axlearn_b200.ops import cuda_ops

            cuda_ops.reserve_sms_for_comm(COMM_SMS)

    def prefetch(self, i: int) -> None:
        if not self.sharded or i in self._ready or not 0 <= i < self._num_layers:
            return
        if self._stream is None:
            self._ready[i] = ([gather_leaf(t[i], p) for t, p in zip(self._leaves, self._plans)], None)
            return
        cur = torch.cuda.current_stream(self._device)
        self._stream.wait_stream(cur)
        with torch.cuda.stream(self._stream):
            full = [gather_leaf(t[i].detach(), p) for t, p in zip(self._leaves, self._plans)]
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._ready[i] = (full, ev)

    def get(self, i: int) -> list[torch.Tensor]:
        """Full tensors of layer ``i`` in leaf order (blocks the current stream until the
        gather has landed)."""
        if not self.sharded:
            return [t[i] for t in self._leaves]
        self.prefetch(i)
        full, ev = self._ready.pop(i)
        if ev is not None:
            torch.cuda.current_stream(self._device).wait_event(ev)
            for t in full:
                t.record_stream(torch.cuda.current_stream(self._device))
        return full

    def scatter_grads(self, i: int, full_grads: Sequence[Optional[torch.Tensor]]) -> None:
        """Reduces layer ``i``'s full gradients to shards and accumulates them into
        ``stacked.grad[i]``, asynchronously on the comm stream."""
        if self._stream is None:
            for t, p, g in zip(self._leaves, self._plans, full_grads):
                if g is not None:
                    accumulate_grad_slice(t, i, scatter_grad_leaf(g, p))
            return
        cur = torch.cuda.current_stream(self._device)
        self._stream.wait_stream(cur)
        with torch.cuda.stream(self._stream):
            for t, p, g in zip(self._leaves, self._plans, full_grads):
                if g is None:
                    continue
                g.record_stream(self._stream)
                accumulate_grad_slice(t, i, scatter_grad_leaf(g, p))
