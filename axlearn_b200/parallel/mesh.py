"""Named device mesh for a one-process-per-GPU job.

The reference describes parallelism with a logical mesh whose axes are
``("pipeline", "data", "expert", "fsdp", "seq", "model")`` and lets a compiler place
collectives (axlearn/experiments/text/gpt/common.py:80,158-188; axlearn/common/utils.py:
85-116, 1874-2025; mesh rules at axlearn/common/trainer.py:142-152,1414-1436).  Here the mesh
is a rank → coordinate map: every rank owns exactly one GPU, each mesh axis (or tuple of
axes) maps to a ``torch.distributed`` process group, and layers issue their collectives
explicitly on those groups (or on fused peer-memory kernels that are handed the group's
ranks).  A mesh can also be built over *fake* ranks, without any process group, to test the
shape logic on a single CPU.

Axis order is major → minor: the last axis varies fastest across consecutive ranks, so the
most communication-intensive axes (``model``, ``seq``, ``fsdp``) land on neighbouring GPUs
of one NVSwitch domain while ``data`` / ``pipeline`` span nodes.
"""

from __future__ import annotations

import dataclasses
import math
import re
import threading
from typing import Any, Optional, Sequence, Union

import numpy as np
import torch
import torch.distributed as dist

MeshShape = Sequence[int]

CANONICAL_AXIS_NAMES = ("pipeline", "data", "expert", "fsdp", "seq", "model")


@dataclasses.dataclass
class HybridMeshShape:
    """``ici_mesh_shape``: per-axis extent inside one NVLink domain (node);
    ``dcn_mesh_shape``: per-axis extent across nodes.  Global extent = product."""

    ici_mesh_shape: MeshShape
    dcn_mesh_shape: MeshShape

    __config_value__ = True

    def __post_init__(self):
        if len(self.ici_mesh_shape) != len(self.dcn_mesh_shape):
            raise ValueError(
                f"ici {self.ici_mesh_shape} and dcn {self.dcn_mesh_shape} must have the same rank"
            )

    def __len__(self):
        return len(self.ici_mesh_shape)


def mesh_shape_from_axes(
    *,
    pipeline: int = 1,
    data: int = 1,
    expert: int = 1,
    fsdp: int = 1,
    seq: int = 1,
    model: int = 1,
) -> tuple[int, ...]:
    """Builds a canonical 6-axis mesh shape; at most one axis may be ``-1`` (inferred)."""
    return (pipeline, data, expert, fsdp, seq, model)


def infer_mesh_shape(mesh_shape: MeshShape, *, num_devices: int) -> tuple[int, ...]:
    """Resolves a single ``-1`` entry from the device count."""
    shape = tuple(int(s) for s in mesh_shape)
    holes = [i for i, s in enumerate(shape) if s == -1]
    if len(holes) > 1:
        raise ValueError(f"At most one axis may be -1: {shape}")
    if not holes:
        if math.prod(shape) != num_devices and num_devices is not None:
            # Leave validation to the caller: some callers pick a sub-mesh.
            pass
        return shape
    known = math.prod(s for s in shape if s != -1)
    if known == 0 or num_devices % known != 0:
        raise ValueError(f"Cannot infer -1 in {shape} for {num_devices} devices")
    out = list(shape)
    out[holes[0]] = num_devices // known
    return tuple(out)


def build_device_grid(
    mesh_shape: Union[MeshShape, HybridMeshShape],
    *,
    num_devices: int,
    devices_per_node: int = 8,
) -> np.ndarray:
    """Returns an int array of global ranks with shape ``mesh_shape``.

    Plain shapes spanning several nodes are split like the reference does: the first
    non-singleton axis divisible by the number of nodes is laid across nodes (DCN), the rest
    stays inside a node.  Hybrid shapes state the split explicitly.
    """
    num_nodes = max(1, num_devices // devices_per_node) if num_devices > devices_per_node else 1
    if isinstance(mesh_shape, HybridMeshShape):
        ici = infer_mesh_shape(mesh_shape.ici_mesh_shape, num_devices=num_devices // num_nodes)
        dcn = infer_mesh_shape(mesh_shape.dcn_mesh_shape, num_devices=num_nodes)
    else:
        shape = infer_mesh_shape(mesh_shape, num_devices=num_devices)
        if math.prod(shape) != num_devices:
            raise ValueError(f"mesh {shape} does not cover {num_devices} devices")
        if num_nodes == 1:
            return np.arange(num_devices, dtype=np.int64).reshape(shape)
        dcn = [1] * len(shape)
        ici = list(shape)
        for i, s in enumerate(shape):
            if s != 1 and s % num_nodes == 0:
                dcn[i] = num_nodes
                ici[i] = s // num_nodes
                break
        else:
            raise ValueError(f"No axis of {shape} is divisible by the node count {num_nodes}")
    if math.prod(ici) * math.prod(dcn) != num_devices:
        raise ValueError(f"ici {ici} x dcn {dcn} does not cover {num_devices} devices")
    per_node = math.prod(ici)
    n = len(ici)
    # ranks[node, local] -> reshape to (dcn..., ici...) -> interleave to (d0,i0,d1,i1,...).
    ranks = np.arange(num_devices, dtype=np.int64).reshape(tuple(dcn) + tuple(ici))
    perm = []
    for i in range(n):
        perm += [i, n + i]
    ranks = ranks.transpose(perm).reshape([d * c for d, c in zip(dcn, ici)])
    del per_node
    return ranks


AxisSpec = Union[None, str, Sequence[str]]


def _axes_tuple(axes: AxisSpec) -> tuple[str, ...]:
    if axes is None:
        return ()
    if isinstance(axes, str):
        return (axes,)
    return tuple(a for a in axes if a is not None)


class Mesh:
    """A named grid of ranks plus the process groups derived from it."""

    def __init__(
        self,
        ranks: np.ndarray,
        axis_names: Sequence[str],
        *,
        rank: Optional[int] = None,
        create_groups: Optional[bool] = None,
    ):
        ranks = np.asarray(ranks)
        if ranks.ndim != len(axis_names):
            raise ValueError(f"mesh rank {ranks.ndim} != len(axis_names) {len(axis_names)}")
        if len(set(axis_names)) != len(axis_names):
            raise ValueError(f"duplicate axis names {axis_names}")
        self.ranks = ranks
        self.axis_names = tuple(axis_names)
        if rank is None:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        self.rank = int(rank)
        where = np.argwhere(ranks == self.rank)
        if len(where) != 1:
            raise ValueError(f"rank {self.rank} does not appear exactly once in the mesh")
        self.coords = dict(zip(self.axis_names, (int(c) for c in where[0])))
        if create_groups is None:
            create_groups = dist.is_available() and dist.is_initialized() and ranks.size > 1
        self._real = bool(create_groups)
        self._groups: dict[tuple[str, ...], Any] = {}
        self._group_ranks: dict[tuple[str, ...], list[int]] = {}

    # ------------------------------------------------------------------ shape queries
    @property
    def shape(self) -> dict[str, int]:
        return dict(zip(self.axis_names, self.ranks.shape))

    @property
    def size(self) -> int:
        return int(self.ranks.size)

    def axis_size(self, axes: AxisSpec) -> int:
        return math.prod(self.shape[a] for a in _axes_tuple(axes)) if _axes_tuple(axes) else 1

    def axis_index(self, axes: AxisSpec) -> int:
        """Linear index of this rank along ``axes`` (first axis is most significant)."""
        idx = 0
        for a in _axes_tuple(axes):
            idx = idx * self.shape[a] + self.coords[a]
        return idx

    def present_axes(self, axes: AxisSpec) -> tuple[str, ...]:
        """Subset of ``axes`` that exist in this mesh with extent > 1."""
        return tuple(a for a in _axes_tuple(axes) if a in self.shape and self.shape[a] > 1)

    def ranks_along(self, axes: AxisSpec, *, coords: Optional[dict[str, int]] = None) -> list[int]:
        """Global ranks of the group that varies ``axes`` and fixes all other coordinates
        at this rank's (or ``coords``) values, ordered by axis_index."""
        axes_t = _axes_tuple(axes)
        coords = coords or self.coords
        index = []
        for name in self.axis_names:
            index.append(slice(None) if name in axes_t else coords[name])
        sub = self.ranks[tuple(index)]
        kept = [n for n in self.axis_names if n in axes_t]
        sub = np.transpose(sub, [kept.index(a) for a in axes_t]) if len(axes_t) > 1 else sub
        return [int(r) for r in np.asarray(sub).reshape(-1)]

    # ------------------------------------------------------------------ process groups
    def group(self, axes: AxisSpec):
        """Process group spanning ``axes`` for this rank; ``None`` when the group is
        trivial (size 1) or the mesh is fake."""
        axes_t = tuple(a for a in _axes_tuple(axes) if a in self.shape)
        if self.axis_size(axes_t) == 1 or not self._real:
            return None
        if axes_t in self._groups:
            return self._groups[axes_t]
        # new_group is collective over the world: every rank creates every sibling group in
        # the same order and keeps the one it belongs to.
        mine = None
        other_names = [n for n in self.axis_names if n not in axes_t]
        other_shape = [self.shape[n] for n in other_names]
        for flat in range(math.prod(other_shape) if other_shape else 1):
            oc = np.unravel_index(flat, other_shape) if other_shape else ()
            coords = dict(zip(other_names, (int(c) for c in oc)))
            coords.update({a: 0 for a in axes_t})
            members = self.ranks_along(axes_t, coords=coords)
            g = dist.new_group(ranks=members)
            if self.rank in members:
                mine = g
                self._group_ranks[axes_t] = members
        self._groups[axes_t] = mine
        return mine

    def group_ranks(self, axes: AxisSpec) -> list[int]:
        return self.ranks_along(tuple(a for a in _axes_tuple(axes) if a in self.shape))

    # ------------------------------------------------------------------ sharding math
    def shard_shape(self, shape: Sequence[int], mesh_axes: Optional[Sequence[AxisSpec]]) -> tuple:
        """Local shape of a tensor of global ``shape`` partitioned by ``mesh_axes``."""
        if mesh_axes is None:
            return tuple(shape)
        if len(mesh_axes) != len(shape):
            raise ValueError(f"mesh_axes {mesh_axes} do not match shape {tuple(shape)}")
        out = []
        for dim, axes in zip(shape, mesh_axes):
            n = self.axis_size(self.present_axes(axes))
            if dim % n != 0:
                raise ValueError(f"dim {dim} of {tuple(shape)} is not divisible by {axes}={n}")
            out.append(dim // n)
        return tuple(out)

    def shard_slices(
        self, shape: Sequence[int], mesh_axes: Optional[Sequence[AxisSpec]]
    ) -> tuple[slice, ...]:
        """Index of this rank's shard inside the global tensor."""
        if mesh_axes is None:
            return tuple(slice(0, d) for d in shape)
        out = []
        for dim, axes in zip(shape, mesh_axes):
            present = self.present_axes(axes)
            n = self.axis_size(present)
            i = self.axis_index(present)
            out.append(slice(i * (dim // n), (i + 1) * (dim // n)))
        return tuple(out)

    def replica_id(self, mesh_axes: Optional[Sequence[AxisSpec]]) -> int:
        """0 for exactly one rank among those that hold the same shard (the writer)."""
        used = set()
        for axes in mesh_axes or ():
            used.update(self.present_axes(axes))
        rid = 0
        for name in self.axis_names:
            if name not in used:
                rid = rid * self.shape[name] + self.coords[name]
        return rid

    # ------------------------------------------------------------------ context manager
    def __enter__(self):
        _mesh_tls.stack.append(self)
        return self

    def __exit__(self, *exc):
        _mesh_tls.stack.pop()

    def __repr__(self):
        return f"Mesh({self.shape}, rank={self.rank}, coords={self.coords})"


class _MeshStack(threading.local):
    def __init__(self):
        self.stack: list[Mesh] = []


_mesh_tls = _MeshStack()


def current_mesh() -> Optional[Mesh]:
    return _mesh_tls.stack[-1] if _mesh_tls.stack else None


def single_device_mesh(axis_names: Sequence[str] = CANONICAL_AXIS_NAMES) -> Mesh:
    return Mesh(np.zeros([1] * len(axis_names), dtype=np.int64), axis_names, rank=0)


def create_mesh(
    mesh_shape: Union[MeshShape, HybridMeshShape],
    axis_names: Sequence[str],
    *,
    world_size: Optional[int] = None,
    rank: Optional[int] = None,
    devices_per_node: int = 8,
    create_groups: Optional[bool] = None,
) -> Mesh:
    if world_size is None:
        world_size = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    grid = build_device_grid(mesh_shape, num_devices=world_size, devices_per_node=devices_per_node)
    return Mesh(grid, axis_names, rank=rank, create_groups=create_groups)


def select_mesh_rule(
    mesh_selector: str, mesh_rules: Optional[Sequence[tuple[str, Any]]]
) -> tuple[bool, Any]:
    """First rule whose regex fully matches the selector: ``(matched, value)``."""
    for regex, value in mesh_rules or ():
        if re.fullmatch(regex, mesh_selector):
            return True, value
    return False, None
