"""Gradient reductions that a one-process-per-GPU runtime must issue itself.

The reference differentiates one global program, so every gradient comes out already summed
over the batch and sharded like its parameter.  Here each rank differentiates its own slice
of the batch; this file supplies what is still missing afterwards:

* ``sync_grads``: a parameter that is *not* storage-sharded over some batch axis (``data``,
  or ``fsdp`` for small replicated tensors such as norm scales) holds only this rank's
  partial gradient; it is summed over exactly the batch axes its spec does not mention.
  (Storage-sharded leaves of repeated layers were already reduce-scattered by the FSDP path.)
* ``sharded_sum_of_squares``: global squared norm over a sharded tree counting each element
  once, for ``clip_by_global_norm`` (axlearn/common/optimizers.py:1149-1184 in the reference).
"""

from __future__ import annotations

from typing import Any, Optional, Sequence

import torch
import torch.distributed as dist

from axlearn_b200.common.utils import TensorSpec, flatten_items
from axlearn_b200.parallel.mesh import Mesh, current_mesh

BATCH_AXES = ("data", "expert", "fsdp", "seq")
# Parameters replicated over the pipeline axis (embeddings, final norm, head) receive a part of
# their gradient on every stage (see common/pipeline.py), so it is summed over that axis too.
REDUCE_AXES = BATCH_AXES + ("pipeline",)


def _axes_in_spec(mesh_axes: Optional[Sequence[Any]]) -> set:
    used: set = set()
    for entry in mesh_axes or ():
        if entry is None:
            continue
        used.update((entry,) if isinstance(entry, str) else tuple(a for a in entry if a))
    return used


def _spec_list(tree: Any, specs: Optional[Any]) -> list:
    leaves = flatten_items(tree)
    if specs is None:
        return [None] * len(leaves)
    spec_map = dict(flatten_items(specs, is_leaf=lambda x: isinstance(x, TensorSpec)))
    return [spec_map.get(path) for path, _ in leaves]


def sync_grads(grads: Any, *, specs: Any, mesh: Optional[Mesh] = None, skip_storage_sharded: bool = True) -> None:
    """In place: sums each gradient over the batch axes that do not shard its parameter."""
    mesh = mesh or current_mesh()
    if mesh is None or mesh.size == 1:
        return
    for (path, g), spec in zip(flatten_items(grads), _spec_list(grads, specs)):
        if g is None:
            continue
        used = _axes_in_spec(spec.mesh_axes if spec is not None else None)
        missing = tuple(a for a in mesh.present_axes(REDUCE_AXES) if a not in used)
        if not missing:
            continue
        group = mesh.group(missing)
        if group is not None:
            dist.all_reduce(g, group=group)


def sharded_sum_of_squares(tree: Any, *, specs: Optional[Any] = None, mesh: Optional[Mesh] = None) -> torch.Tensor:
    """Sum of squares over the *global* tensors described by ``tree`` + ``specs``."""
    mesh = mesh or current_mesh()
    leaves = [(p, t) for p, t in flatten_items(tree) if isinstance(t, torch.Tensor)]
    if not leaves:
        return torch.zeros(())
    device = leaves[0][1].device
    from axlearn_b200.ops import dispatch

    use_kernel = device.type == "cuda" and not dispatch._flags.force_reference  # pylint: disable=protected-access
    weights = [1.0] * len(leaves)
    if mesh is not None and mesh.size > 1:
        spec_map = dict(zip([p for p, _ in flatten_items(tree)], _spec_list(tree, specs)))
        for i, (path, _) in enumerate(leaves):
            spec = spec_map.get(path)
            used = _axes_in_spec(spec.mesh_axes if spec is not None else None)
            shard_ways = mesh.axis_size(mesh.present_axes(tuple(used)))
            weights[i] = 1.0 / (mesh.size // max(1, shard_ways))
    if use_kernel:
        total = dispatch._ops().sum_of_squares([t for _, t in leaves], weights)  # pylint: disable=protected-access
    else:
        total = torch.zeros((), dtype=torch.float32, device=device)
        for (_, t), w in zip(leaves, weights):
            total = total + t.float().pow(2).sum() * w
    if mesh is not None and mesh.size > 1 and mesh._real:  # pylint: disable=protected-access
        total = total.clone()
        dist.all_reduce(total)
    return total
