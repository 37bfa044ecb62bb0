"""Pipeline parallelism: stages on different ranks, micro-batches streamed between them.

Parity targets in the reference: ``Pipeline`` with ``GPipeSchedule`` (axlearn/common/pipeline.py:
197-355, 421-661: stage parameters stacked ``[num_stages, ...]`` and sharded over the
``pipeline`` mesh axis, ``M + N - 1`` ticks of a vmapped stage function with a shift between
stages) and ``PipelinedTransformerLayer`` (axlearn/common/attention.py:4458-4551).

Here a stage is simply the code a rank runs: rank ``s`` of the ``pipeline`` axis owns slice ``s``
of the stacked stage parameters, receives each micro-batch's activations from rank ``s - 1``
with a point-to-point ``recv``, runs its stage and ``send``s the result on -- the GPipe schedule
(all micro-batches forward, then all backward) falls out of autograd: ``recv`` / ``send`` are
autograd functions whose backward passes are the matching ``send`` / ``recv`` of gradients, and
the engine replays them in reverse order on every rank.  Point-to-point transfers stay on the
library (NCCL / gloo) as stage boundaries are bandwidth-light.

After the last stage the output is broadcast over the ``pipeline`` group so that the rest of the
model (final norm, head, loss) runs identically on every rank; the backward of that broadcast
*sums* the ranks' output gradients onto the last stage, and the trainer scales the loss by
``1 / num_stages`` so that the sum is the true gradient (and gradients of parameters replicated
over the ``pipeline`` axis, which are all-reduced, come out right as well).

Without a ``pipeline`` mesh axis the stages simply run one after the other on the local rank,
which is the oracle in tests.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Optional

import torch
import torch.distributed as dist

from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.module import current_context, new_output_collection, nowrap, set_current_context
from axlearn_b200.common.utils import VDict, flatten_items, tree_map
from axlearn_b200.parallel import collectives as coll
from axlearn_b200.parallel.mesh import current_mesh

Tensor = torch.Tensor


def _pipeline_group():
    """(group, size, index, global ranks in stage order) of the ``pipeline`` axis."""
    mesh = current_mesh()
    if mesh is None or mesh.shape.get("pipeline", 1) == 1:
        return None, 1, 0, [0]
    return mesh.group("pipeline"), mesh.shape["pipeline"], mesh.coords["pipeline"], mesh.ranks_along("pipeline")


class _Send(torch.autograd.Function):
    """Sends ``x`` to global rank ``dst``; returns a token that keeps the node in the graph.
    Backward receives the gradient of ``x`` from ``dst``."""

    @staticmethod
    def forward(ctx, x, dst, group):
        ctx.dst, ctx.group, ctx.meta = dst, group, (x.shape, x.dtype, x.device)
        dist.send(x.contiguous(), dst=dst, group=group)
        return x.new_zeros(())

    @staticmethod
    def backward(ctx, _token_grad):
        shape, dtype, device = ctx.meta
        g = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(g, src=ctx.dst, group=ctx.group)
        return g, None, None


class _Recv(torch.autograd.Function):
    """Receives a tensor like ``like`` from global rank ``src``; backward sends the gradient
    back.  ``anchor`` (a tensor that requires grad) ties the node into the graph."""

    @staticmethod
    def forward(ctx, anchor, src, group, shape, dtype):
        ctx.src, ctx.group = src, group
        out = torch.empty(shape, dtype=dtype, device=anchor.device)
        dist.recv(out, src=src, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        dist.send(g.contiguous(), dst=ctx.src, group=ctx.group)
        return None, None, None, None, None


class _BroadcastFromLast(torch.autograd.Function):
    """Forward: every rank gets the last stage's ``y``.  Backward: the ranks' gradients are summed
    onto the last stage.  ``tokens`` are the send tokens of this rank (kept alive in the graph)."""

    @staticmethod
    def forward(ctx, y, src, group, is_last, *tokens):
        ctx.src, ctx.group, ctx.is_last, ctx.n = src, group, is_last, len(tokens)
        out = y.detach().clone().contiguous()
        dist.broadcast(out, src=src, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.reduce(g, dst=ctx.src, op=dist.ReduceOp.SUM, group=ctx.group)
        zero = g.new_zeros(())
        return (g if ctx.is_last else torch.zeros_like(g)), None, None, None, *([zero] * ctx.n)


class Pipeline(BaseLayer):
    """``num_stages`` copies of ``layer`` applied in sequence, one per rank of the ``pipeline``
    axis, over ``num_microbatches`` slices of the batch."""

    @config_class
    class Config(BaseLayer.Config):
        layer: Required[InstantiableConfig] = REQUIRED
        num_layers: Required[int] = REQUIRED          # number of stages (the reference's name)
        num_microbatches: Required[int] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("layer", cfg.layer)

    # ------------------------------------------------------------------ parameters
    @nowrap
    def create_parameter_specs_recursively(self):
        n = self._config.num_layers

        def stack(spec: ParameterSpec) -> ParameterSpec:
            axes = (coll.ComputeAxis("pipeline"),) + tuple(spec.mesh_axes or (None,) * len(spec.shape))
            return dataclasses.replace(spec, shape=(n,) + tuple(spec.shape), mesh_axes=axes)

        inner = self.layer.create_parameter_specs_recursively()
        # A plain dict (not a VDict): the trainer reserves VDict for stacks whose gradients are
        # written slice by slice by the layer loop; stage gradients arrive through autograd.
        return {"layer": tree_map(stack, inner, is_leaf=lambda x: isinstance(x, ParameterSpec))}

    @nowrap
    def initialize_parameters_recursively(self, prng_key, *, prebuilt=None, device=None):
        """Every stage is initialised from its own key; a rank keeps only its own stage(s)."""
        n = self._config.num_layers
        _, size, index, _ = _pipeline_group()
        (child_key,) = prng.split(prng_key, 1)
        keys = prng.split(child_key, n)
        per_rank = n // size
        mine = range(index * per_rank, (index + 1) * per_rank)
        stages = [self.layer.initialize_parameters_recursively(keys[i], device=device) for i in mine]
        return {"layer": tree_map(lambda *ts: torch.stack(ts, dim=0), *stages)}

    # ------------------------------------------------------------------ execution
    def _run_stage(self, local_index: int, global_index: int, x: Tensor, kwargs: dict) -> Tensor:
        ctx = current_context()
        params = tree_map(lambda t: t[local_index], ctx.state["layer"])
        key = None if ctx.prng_key is None else prng.fold_in(ctx.prng_key, global_index)
        oc = ctx.output_collection.get_or_add_child(f"stage{global_index}")
        stage_ctx = dataclasses.replace(ctx, state={"layer": params}, prng_key=key, output_collection=oc)
        with set_current_context(stage_ctx, require_parent=False):
            out = self.layer(x, **kwargs)
        return out.data if hasattr(out, "data") and not isinstance(out, Tensor) else out

    def forward(self, data: Tensor, **kwargs) -> Tensor:
        cfg = self._config
        group, size, index, ranks = _pipeline_group()
        n, m = cfg.num_layers, cfg.num_microbatches
        if n % size:
            raise ValueError(f"{n} stages cannot be split over a pipeline axis of {size}")
        per_rank = n // size
        if data.shape[0] % m:
            raise ValueError(f"batch {data.shape[0]} is not divisible into {m} micro-batches")
        micro = list(data.chunk(m, dim=0))
        # Per-microbatch keyword tensors (e.g. segment ids) are split alike.
        kw_micro = [
            {k: (v.chunk(m, dim=0)[i] if isinstance(v, Tensor) and v.dim() > 0 and v.shape[0] == data.shape[0] else v)
             for k, v in kwargs.items()} for i in range(m)]
        is_first, is_last = index == 0, index == size - 1
        outs, tokens = [], []
        anchor = next((t for _, t in flatten_items(current_context().state["layer"]) if t.requires_grad), None)
        for i in range(m):
            if is_first:
                x = micro[i]
            else:
                recv_anchor = anchor if anchor is not None else micro[i]
                x = _Recv.apply(recv_anchor, ranks[index - 1], group, micro[i].shape, micro[i].dtype)
            for j in range(per_rank):
                x = self._run_stage(j, index * per_rank + j, x, kw_micro[i])
            if is_last:
                outs.append(x)
            else:
                tokens.append(_Send.apply(x, ranks[index + 1], group))
        if size == 1:
            return torch.cat(outs, dim=0)
        y = torch.cat(outs, dim=0) if is_last else torch.zeros_like(data)
        return _BroadcastFromLast.apply(y, ranks[-1], group, is_last, *tokens)


def loss_scale_for_pipeline() -> float:
    """Factor the trainer applies to the loss before ``backward`` (see the module docstring)."""
    return 1.0 / _pipeline_group()[1]


def _pipelined_transformer_layer():
    """Defined lazily to keep ``attention`` free of an import cycle."""
    from axlearn_b200.common.attention import BaseStackedTransformerLayer, StackedTransformerLayer

    class PipelinedTransformerLayer(BaseStackedTransformerLayer):
        """``num_layers`` transformer layers split into ``num_stages`` pipeline stages of
        ``num_layers / num_stages`` layers each (child ``pipeline`` -> ``layer`` = a stacked
        transformer), run over ``num_microbatches`` micro-batches."""

        @config_class
        class Config(BaseStackedTransformerLayer.Config):
            num_stages: Required[int] = REQUIRED
            num_microbatches: Required[int] = REQUIRED
            stage: InstantiableConfig = StackedTransformerLayer.default_config()
            pipeline: InstantiableConfig = Pipeline.default_config()

        def __init__(self, cfg, *, parent=None):
            super().__init__(cfg, parent=parent)
            if cfg.num_layers % cfg.num_stages:
                raise ValueError(f"num_stages {cfg.num_stages} must divide num_layers {cfg.num_layers}")
            stage = cfg.stage.clone(input_dim=cfg.input_dim, num_layers=cfg.num_layers // cfg.num_stages, layer=cfg.layer)
            self._add_child("pipeline", cfg.pipeline.clone(
                layer=stage, num_layers=cfg.num_stages, num_microbatches=cfg.num_microbatches))

        def forward(self, data, **kwargs):
            return self.Output(data=self.pipeline(data, **kwargs), self_attention_probs=None,
                               self_attention_kv_state=None, cross_attention_probs=None)

    return PipelinedTransformerLayer


PipelinedTransformerLayer = _pipelined_transformer_layer()
