"""Autograd-aware collectives on mesh axes.

Every function takes mesh axis names, looks up the process group on the mesh in scope and
degenerates to the identity when that group is trivial — so the same layer code runs on one
device, on CPU/gloo ranks in tests, and on NCCL ranks.  These are the *baseline* collectives
(one library call each); the fused peer-memory kernels in ``axlearn_b200.ops`` replace the
hot ones and are validated against these.

The reference never spells these out: XLA's SPMD partitioner inserts them from sharding
annotations (axlearn/common/utils.py:637-700 ``with_sharding_constraint``/``maybe_shard``);
the explicit ones it does write are in axlearn/common/mixture_of_experts.py:2139-2210,
2670-2726.
"""

from __future__ import annotations

import contextlib
import threading
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from axlearn_b200.parallel.mesh import AxisSpec, Mesh, current_mesh


def _group(axes: AxisSpec, mesh: Optional[Mesh] = None):
    mesh = mesh or current_mesh()
    if mesh is None:
        return None, 1, 0
    present = mesh.present_axes(axes)
    if not present:
        return None, 1, 0
    return mesh.group(present), mesh.axis_size(present), mesh.axis_index(present)


def axis_size(axes: AxisSpec) -> int:
    return _group(axes)[1]


def axis_index(axes: AxisSpec) -> int:
    return _group(axes)[2]


def current_group(axes: AxisSpec):
    """Process group of ``axes`` on the current mesh (None when the axes have extent 1)."""
    return _group(axes)[0]


# ------------------------------------------------------------------------------------------
# Raw (non-differentiable) helpers.
# ------------------------------------------------------------------------------------------


@torch.no_grad()
def all_gather_raw(x: torch.Tensor, group, world: int, dim: int = 0) -> torch.Tensor:
    """Concatenation over the group's ranks along ``dim``."""
    x = x.contiguous()
    if x.dim() == 0:
        x = x.reshape(1)
    flat = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(flat, x, group=group)
    if dim == 0:
        return flat
    # [W*d0, ...] -> [W, d0, ..., d, ...] -> [d0, ..., W*d, ...]
    out = flat.reshape((world,) + tuple(x.shape)).movedim(0, dim)
    shape = list(x.shape)
    shape[dim] *= world
    return out.reshape(shape)


@torch.no_grad()
def reduce_scatter_raw(x: torch.Tensor, group, world: int, dim: int = 0) -> torch.Tensor:
    """Sum over the group, each rank keeping its slice along ``dim``."""
    if dim != 0:
        # [..., W*d, ...] -> [W, ..., d, ...] -> [W * d0, ...] (rank-major rows).
        shape = list(x.shape)
        x = x.reshape(shape[:dim] + [world, shape[dim] // world] + shape[dim + 1 :]).movedim(dim, 0)
        x = x.contiguous()
        x = x.reshape((-1,) + tuple(x.shape[2:]))
    x = x.contiguous()
    out = torch.empty((x.shape[0] // world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


# ------------------------------------------------------------------------------------------
# Differentiable collectives.
# ------------------------------------------------------------------------------------------


class _AllReduce(torch.autograd.Function):
    """y = sum over group; dy passes through (the "g" operator of tensor parallelism)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _IdentityFwdAllReduceBwd(torch.autograd.Function):
    """y = x; dx = sum over group of dy (the "f" operator of tensor parallelism)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _AllGather(torch.autograd.Function):
    """Concatenate shards on ``dim``; backward reduce-scatters (sums) the gradient."""

    @staticmethod
    def forward(ctx, x, group, world, dim):
        ctx.group, ctx.world, ctx.dim = group, world, dim
        return all_gather_raw(x, group, world, dim)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_raw(g, ctx.group, ctx.world, ctx.dim), None, None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world, dim):
        ctx.group, ctx.world, ctx.dim = group, world, dim
        return reduce_scatter_raw(x, group, world, dim)

    @staticmethod
    def backward(ctx, g):
        return all_gather_raw(g, ctx.group, ctx.world, ctx.dim), None, None, None


class _AllToAll(torch.autograd.Function):
    """Splits ``split_dim`` into ``world`` pieces, sends piece r to rank r, concatenates what
    arrives on ``concat_dim``."""

    @staticmethod
    def forward(ctx, x, group, world, split_dim, concat_dim):
        ctx.args = (group, world, split_dim, concat_dim)
        return _all_to_all_raw(x, group, world, split_dim, concat_dim)

    @staticmethod
    def backward(ctx, g):
        group, world, split_dim, concat_dim = ctx.args
        return _all_to_all_raw(g, group, world, concat_dim, split_dim), None, None, None, None


def _all_to_all_raw(x, group, world, split_dim, concat_dim):
    parts = [p.contiguous() for p in x.chunk(world, dim=split_dim)]
    outs = [torch.empty_like(parts[0]) for _ in range(world)]
    if dist.get_backend(group) == "gloo":
        # gloo has no all-to-all: gather everything and keep the pieces addressed to this rank.
        stacked = torch.stack(parts, dim=0)
        everyone = [torch.empty_like(stacked) for _ in range(world)]
        dist.all_gather(everyone, stacked, group=group)
        me = dist.get_rank(group)
        outs = [everyone[r][me] for r in range(world)]
    else:
        dist.all_to_all(outs, parts, group=group)
    return torch.cat(outs, dim=concat_dim)


def psum(x: torch.Tensor, axes: AxisSpec) -> torch.Tensor:
    """Sum over ``axes``; gradient passes through unchanged."""
    group, world, _ = _group(axes)
    if world == 1:
        return x
    from axlearn_b200.parallel import peer_allreduce

    if peer_allreduce.usable(x, group, world):
        return peer_allreduce.psum(x, group)
    return _AllReduce.apply(x, group)


def psum_grad(x: torch.Tensor, axes: AxisSpec) -> torch.Tensor:
    """Identity whose *gradient* is summed over ``axes``."""
    group, world, _ = _group(axes)
    if world == 1:
        return x
    from axlearn_b200.parallel import peer_allreduce

    if peer_allreduce.usable(x, group, world):
        return peer_allreduce.psum_grad(x, group)
    return _IdentityFwdAllReduceBwd.apply(x, group)


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, axes: AxisSpec) -> Optional[torch.Tensor]:
    """``psum(x @ w, axes)`` with the reduction's stores fused into the GEMM epilogue (peer
    memory), or None when that path does not apply."""
    group, world, _ = _group(axes)
    if world == 1 or _tp_seq.dim is not None:
        return None
    from axlearn_b200.parallel import peer_allreduce

    return peer_allreduce.row_parallel_linear(x, w, group, world)


def all_gather(x: torch.Tensor, axes: AxisSpec, *, dim: int = 0) -> torch.Tensor:
    group, world, _ = _group(axes)
    if world == 1:
        return x
    return _AllGather.apply(x, group, world, dim % x.dim())


# ------------------------------------------------------------------------------------------
# Sequence-sharded tensor-parallel regions ("Megatron sequence parallelism").
#
# Between the tensor-parallel blocks of a transformer layer (norms, residual adds, dropout) every
# rank of the `model` axis would otherwise hold and process the same [B, T, D] activations.  With
# the mode on, those regions work on a 1 / tp slice of the sequence: a column-parallel linear
# all-gathers its input (backward: reduce-scatter of the input gradient) and a row-parallel linear
# reduce-scatters its output (backward: all-gather) -- the same bytes as the all-reduce pair they
# replace.  The mode is a thread-local flag set INSIDE a layer's forward, so that a rematerialised
# forward in the backward pass sees it too.
# ------------------------------------------------------------------------------------------


class _TpSeqState(threading.local):
    def __init__(self):
        self.dim: Optional[int] = None


_tp_seq = _TpSeqState()


@contextlib.contextmanager
def tp_sequence_parallel(enabled: bool = True, *, dim: int = 1):
    prev, _tp_seq.dim = _tp_seq.dim, (dim if enabled else None)
    try:
        yield
    finally:
        _tp_seq.dim = prev


def tp_sequence_parallel_dim() -> Optional[int]:
    return _tp_seq.dim


def tp_enter(x: torch.Tensor, axes: AxisSpec) -> torch.Tensor:
    """Input of a column-parallel linear: the full activations, gradient summed over ``axes``."""
    if _tp_seq.dim is not None:
        return all_gather(x.contiguous(), axes, dim=_tp_seq.dim)
    return psum_grad(x, axes)


def tp_exit(y: torch.Tensor, axes: AxisSpec) -> torch.Tensor:
    """Output of a row-parallel linear: summed over ``axes`` (and sequence-sharded when the mode is on)."""
    if _tp_seq.dim is not None:
        return reduce_scatter(y.contiguous(), axes, dim=_tp_seq.dim)
    return psum(y, axes)


class _ScatterReplicated(torch.autograd.Function):
    """Takes this rank's slice of a tensor that is REPLICATED over the group; the gradient of
    the replicated tensor is the concatenation of the slices' gradients."""

    @staticmethod
    def forward(ctx, x, group, world, dim):
        ctx.group, ctx.world, ctx.dim = group, world, dim
        return x.chunk(world, dim=dim)[dist.get_rank(group)].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_raw(g.contiguous(), ctx.group, ctx.world, ctx.dim), None, None, None


class _GatherReplicated(torch.autograd.Function):
    """All-gathers slices into a tensor whose consumers are replicated over the group: every rank
    computes the same gradient for the whole tensor, so the slice's gradient is just its part."""

    @staticmethod
    def forward(ctx, x, group, world, dim):
        ctx.group, ctx.world, ctx.dim = group, world, dim
        return all_gather_raw(x.contiguous(), group, world, dim)

    @staticmethod
    def backward(ctx, g):
        return g.chunk(ctx.world, dim=ctx.dim)[dist.get_rank(ctx.group)].contiguous(), None, None, None


def scatter_replicated(x: torch.Tensor, axes: AxisSpec, *, dim: int) -> torch.Tensor:
    group, world, _ = _group(axes)
    if world == 1:
        return x
    if x.shape[dim] % world:
        raise ValueError(f"dim {dim} of size {x.shape[dim]} is not divisible by the {world} ranks of {axes}")
    return _ScatterReplicated.apply(x, group, world, dim % x.dim())


def gather_replicated(x: torch.Tensor, axes: AxisSpec, *, dim: int) -> torch.Tensor:
    group, world, _ = _group(axes)
    if world == 1:
        return x
    return _GatherReplicated.apply(x, group, world, dim % x.dim())


def reduce_scatter(x: torch.Tensor, axes: AxisSpec, *, dim: int = 0) -> torch.Tensor:
    group, world, _ = _group(axes)
    if world == 1:
        return x
    return _ReduceScatter.apply(x, group, world, dim % x.dim())


def all_to_all(x: torch.Tensor, axes: AxisSpec, *, split_dim: int, concat_dim: int) -> torch.Tensor:
    group, world, _ = _group(axes)
    if world == 1:
        return x
    return _AllToAll.apply(x, group, world, split_dim % x.dim(), concat_dim % x.dim())


def all_reduce_scalar(x: torch.Tensor, axes: AxisSpec, op: str = "sum") -> torch.Tensor:
    """Non-differentiable reduction of a small tensor (counts, norms, metrics)."""
    group, world, _ = _group(axes)
    if world == 1:
        return x
    y = x.detach().clone()
    dist.all_reduce(y, op={"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op], group=group)
    return y


def barrier(name: str = "") -> None:
    """Cross-process barrier (no-op without an initialised process group)."""
    del name
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def process_index() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def process_count() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


# ------------------------------------------------------------------------------------------
# Parameter un-sharding (FSDP) by partition spec.
# ------------------------------------------------------------------------------------------

# Axes that shard *parameters for storage only*: a layer gathers over them before use.
# "model" (and "pipeline") shard the computation itself and are never gathered.
_COMPUTE_AXES = ("model", "pipeline")


class ComputeAxis(str):
    """A mesh-axis name that, in this partition-spec entry, shards the *computation* and is
    never gathered: e.g. ``ComputeAxis("expert")`` on the expert dim of MoE weights (experts
    live on their rank; tokens travel), while plain ``"expert"`` elsewhere remains a storage
    axis that FSDP gathers."""


def _is_compute_axis(a: str) -> bool:
    return a in _COMPUTE_AXES or isinstance(a, ComputeAxis)


def storage_axes(entry: AxisSpec, mesh: Optional[Mesh] = None) -> tuple[str, ...]:
    mesh = mesh or current_mesh()
    if mesh is None or entry is None:
        return ()
    names = (entry,) if isinstance(entry, str) else tuple(entry)
    return tuple(a for a in mesh.present_axes(names) if not _is_compute_axis(a))


def unshard_param(
    w: torch.Tensor, mesh_axes: Optional[Sequence[AxisSpec]], *, compute_shape: Optional[Sequence[int]] = None
) -> torch.Tensor:
    """Gathers ``w`` over its storage (FSDP) axes; the gradient is reduce-scattered back.

    If ``w`` already has ``compute_shape`` (a prefetcher gathered it ahead of time) it is
    returned as is.
    """
    mesh = current_mesh()
    if mesh is None or mesh_axes is None or mesh.size == 1:
        return w
    if compute_shape is not None and tuple(w.shape) == tuple(compute_shape):
        return w
    for dim, entry in enumerate(mesh_axes):
        axes = storage_axes(entry, mesh)
        if axes:
            w = all_gather(w, axes, dim=dim)
    return w


def compute_shape(shape: Sequence[int], mesh_axes: Optional[Sequence[AxisSpec]]) -> tuple[int, ...]:
    """Shape a parameter has when used in computation: split only over compute axes."""
    mesh = current_mesh()
    if mesh is None or mesh_axes is None:
        return tuple(shape)
    out = []
    for d, entry in zip(shape, mesh_axes):
        names = () if entry is None else ((entry,) if isinstance(entry, str) else tuple(entry))
        comp = tuple(a for a in mesh.present_axes(names) if _is_compute_axis(a))
        out.append(d // mesh.axis_size(comp))
    return tuple(out)


def has_axis(entry: AxisSpec, axis: str) -> bool:
    """True when ``axis`` is named by the spec entry and has extent > 1 on the mesh."""
    mesh = current_mesh()
    if mesh is None or entry is None:
        return False
    names = (entry,) if isinstance(entry, str) else tuple(entry)
    return axis in mesh.present_axes(names)
