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
from axlearn_b200.common.config import REQUIRED, Configurable, InstantiableConfig, Required, config_class
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


class _Transfers:
    """The point-to-point operations of one pipeline pass (forward and its backward).

    Every transfer is posted asynchronously (``isend`` / ``irecv``: on NCCL they run on the
    process group's own streams, beside the compute stream) and waited for only where its data is
    needed, so a stage computes micro-batch ``i`` while micro-batch ``i + 1`` arrives and
    micro-batch ``i - 1`` leaves.  With ``overlap=False`` every operation is waited for at once
    (the plain blocking schedule; kept for debugging).
    """

    def __init__(self, group, overlap: bool):
        self.group = group
        self.overlap = overlap
        self._sends: list = []          # (work, tensor): tensors stay alive until the pass ends
        self._grad_recvs: dict = {}     # micro-batch -> (work, buffer)

    def send(self, x: Tensor, dst: int, *, deferred: bool = False) -> None:
        """``deferred``: never wait here, whatever the mode (the receiver posts its side only after
        its own loop, so waiting would stall both ranks)."""
        x = x.detach().contiguous()
        work = dist.isend(x, dst=dst, group=self.group)
        if self.overlap or deferred:
            self._sends.append((work, x))
        else:
            work.wait()

    def post_recv(self, shape, dtype, device, src: int):
        buf = torch.empty(shape, dtype=dtype, device=device)
        return dist.irecv(buf, src=src, group=self.group), buf

    def grad_from(self, i: int, src: int, meta) -> Tensor:
        """Gradient of micro-batch ``i`` from the next stage.  Backward visits micro-batches in
        reverse order, so the receive for ``i - 1`` is posted before waiting for ``i``."""
        for j in ((i, i - 1) if self.overlap else (i,)):
            if j >= 0 and j not in self._grad_recvs:
                self._grad_recvs[j] = self.post_recv(*meta, src)
        work, buf = self._grad_recvs.pop(i)
        work.wait()
        return buf

    def drain(self) -> None:
        for work, _ in self._sends:
            work.wait()
        self._sends.clear()


class _Sent(torch.autograd.Function):
    """Sends ``x`` (micro-batch ``i``) to global rank ``dst``; returns a token that keeps the node
    in the graph.  Backward receives the gradient of ``x`` from ``dst``."""

    @staticmethod
    def forward(ctx, x, dst, transfers, i):
        ctx.dst, ctx.transfers, ctx.i, ctx.meta = dst, transfers, i, (x.shape, x.dtype, x.device)
        transfers.send(x, dst)
        return x.new_zeros(())

    @staticmethod
    def backward(ctx, _token_grad):
        return ctx.transfers.grad_from(ctx.i, ctx.dst, ctx.meta), None, None, None


class _Received(torch.autograd.Function):
    """Puts a received buffer into the graph; backward sends its gradient back to ``src``.
    ``anchor`` (a tensor that requires grad) ties the node into the graph."""

    @staticmethod
    def forward(ctx, anchor, buf, src, transfers):
        ctx.src, ctx.transfers = src, transfers
        return buf

    @staticmethod
    def backward(ctx, g):
        ctx.transfers.send(g, ctx.src)
        return None, None, None, None


class _BroadcastFromLast(torch.autograd.Function):
    """Forward: every rank gets the last stage's ``y``.  Backward: the ranks' gradients are summed
    onto the last stage.  ``tokens`` are the send tokens of this rank (kept alive in the graph)."""

    @staticmethod
    def forward(ctx, y, src, group, is_last, transfers, *tokens):
        ctx.src, ctx.group, ctx.is_last, ctx.n, ctx.transfers = src, group, is_last, len(tokens), transfers
        transfers.drain()
        out = y.detach().clone().contiguous()
        dist.broadcast(out, src=src, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.reduce(g, dst=ctx.src, op=dist.ReduceOp.SUM, group=ctx.group)
        zero = g.new_zeros(())
        return (g if ctx.is_last else torch.zeros_like(g)), None, None, None, None, *([zero] * ctx.n)


class _CollectStreams(torch.autograd.Function):
    """The output side of the stream schedule.

    Micro-batch ``i`` belongs to stream ``i // (M / N)``, owned by the stage of that index.  The
    last stage has already posted a send of every finished micro-batch to its owner (inside the
    micro-batch loop, so those transfers overlap the remaining compute); here the owners receive
    their streams and one all-gather gives every rank the whole output.  Backward: a
    reduce-scatter sums the ranks' output gradients onto the owners, which return them to the last
    stage -- every rank sends and receives ``1 / N`` of the output instead of the last stage
    serving everything.
    """

    @staticmethod
    def forward(ctx, anchor, group, ranks, index, m, transfers, meta, *outs_or_tokens):
        size = len(ranks)
        per = m // size
        is_last = index == size - 1
        ctx.group, ctx.ranks, ctx.index, ctx.m, ctx.transfers, ctx.meta = group, ranks, index, m, transfers, meta
        ctx.n_inputs = len(outs_or_tokens)
        shape, dtype, device = meta
        if is_last:
            mine = [outs_or_tokens[i].detach() for i in range(index * per, (index + 1) * per)]
        else:
            pending = [transfers.post_recv(shape, dtype, device, ranks[-1]) for _ in range(per)]
            mine = []
            for work, buf in pending:
                work.wait()
                mine.append(buf)
        transfers.drain()
        stream = torch.cat(mine, dim=0).contiguous()
        full = torch.empty((size,) + tuple(stream.shape), dtype=dtype, device=device)
        dist.all_gather_into_tensor(full.view(-1, *stream.shape[1:]), stream, group=group)
        return full.view(-1, *stream.shape[1:])

    @staticmethod
    def backward(ctx, g):
        size, per, index = len(ctx.ranks), ctx.m // len(ctx.ranks), ctx.index
        is_last = index == size - 1
        g = g.contiguous()
        mine = torch.empty((g.shape[0] // size,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(mine, g, op=dist.ReduceOp.SUM, group=ctx.group)
        head = (None,) * 7
        if not is_last:
            for piece in mine.chunk(per, dim=0):
                ctx.transfers.send(piece, ctx.ranks[-1])
            ctx.transfers.drain()
            return head + tuple(g.new_zeros(()) for _ in range(ctx.n_inputs))
        grads: list = [None] * ctx.m
        pending = {}
        for owner in range(size - 1):
            for i in range(owner * per, (owner + 1) * per):
                pending[i] = ctx.transfers.post_recv(*ctx.meta, ctx.ranks[owner])
        for j, piece in enumerate(mine.chunk(per, dim=0)):
            grads[index * per + j] = piece
        for i, (work, buf) in pending.items():
            work.wait()
            grads[i] = buf
        return head + tuple(grads)


class BaseSchedule(Configurable):
    """How micro-batches enter and leave the stages (axlearn/common/pipeline.py:197-661)."""

    @config_class
    class Config(Configurable.Config):
        num_stages: Optional[int] = None         # filled in by ``Pipeline``
        num_microbatches: Optional[int] = None

    @property
    def num_stages(self) -> int:
        return self._config.num_stages

    @property
    def num_microbatches(self) -> int:
        return self._config.num_microbatches

    @property
    def num_iterations(self) -> int:
        """Ticks until the pipeline is flushed."""
        return self.num_microbatches + self.num_stages - 1

    def bubble_fraction(self) -> float:
        return (self.num_stages - 1) / self.num_iterations

    def stage_and_microbatch_at(self, t: int) -> list:
        """``(stage, micro-batch)`` pairs that are busy at tick ``t`` of the forward pass."""
        return [(s, t - s) for s in range(self.num_stages) if 0 <= t - s < self.num_microbatches]

    def output_owner(self, microbatch: int) -> int:
        raise NotImplementedError(type(self))


class GPipeSchedule(BaseSchedule):
    """All inputs live on every stage; all outputs come from the last stage (one broadcast)."""

    def output_owner(self, microbatch: int) -> int:
        return self.num_stages - 1


class StreamSchedule(BaseSchedule):
    """Outputs are kept as ``num_stages`` streams of ``M / N`` micro-batches, one per stage
    (axlearn/common/pipeline.py:421-661): finished micro-batches leave the last stage for their
    owner while later ones are still being computed, and the gradient of the output returns the
    same way, so no stage carries the whole output traffic."""

    def __init__(self, cfg):
        super().__init__(cfg)
        if cfg.num_stages and cfg.num_microbatches and cfg.num_microbatches % cfg.num_stages:
            raise ValueError(f"num_microbatches ({cfg.num_microbatches}) must be divisible by num_stages "
                             f"({cfg.num_stages}) for the stream schedule")

    def output_owner(self, microbatch: int) -> int:
        return microbatch // (self.num_microbatches // self.num_stages)


class Pipeline(BaseLayer):
    """``num_stages`` copies of ``layer`` applied in sequence, one per rank of the ``pipeline``
    axis, over ``num_microbatches`` slices of the batch."""

    @config_class
    class Config(BaseLayer.Config):
        layer: Required[InstantiableConfig] = REQUIRED
        num_layers: Required[int] = REQUIRED          # number of stages (the reference's name)
        num_microbatches: Required[int] = REQUIRED
        schedule: InstantiableConfig = GPipeSchedule.default_config()
        # Post transfers asynchronously and wait where the data is needed (False: blocking).
        overlap_transfers: bool = True

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("layer", cfg.layer)
        self._schedule = cfg.schedule.clone(num_stages=cfg.num_layers, num_microbatches=cfg.num_microbatches).instantiate()

    @property
    def schedule(self) -> BaseSchedule:
        return self._schedule

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
        stream = size > 1 and isinstance(self._schedule, StreamSchedule)
        if stream and m % size:
            raise ValueError(f"{m} micro-batches cannot be kept as {size} equal streams")
        per_stream = m // size if stream else m
        transfers = _Transfers(group, cfg.overlap_transfers)
        outs, tokens = [], []
        anchor = next((t for _, t in flatten_items(current_context().state["layer"]) if t.requires_grad), None)
        meta = (micro[0].shape, micro[0].dtype, micro[0].device)
        incoming = None
        for i in range(m):
            if is_first:
                x = micro[i]
            else:
                work, buf = incoming if incoming is not None else transfers.post_recv(*meta, ranks[index - 1])
                work.wait()
                # The next micro-batch travels while this one is computed.
                incoming = transfers.post_recv(*meta, ranks[index - 1]) if cfg.overlap_transfers and i + 1 < m else None
                x = _Received.apply(anchor if anchor is not None else micro[i], buf, ranks[index - 1], transfers)
            for j in range(per_rank):
                x = self._run_stage(j, index * per_rank + j, x, kw_micro[i])
            if is_last:
                outs.append(x)
                owner = i // per_stream
                if stream and owner != index:
                    transfers.send(x, ranks[owner], deferred=True)
            else:
                tokens.append(_Sent.apply(x, ranks[index + 1], transfers, i))
        if size == 1:
            return torch.cat(outs, dim=0)
        if stream:
            out_meta = (outs[0].shape, outs[0].dtype, outs[0].device) if is_last else None
            out_meta = _share_meta(out_meta, ranks[-1], group, meta)
            link = anchor if anchor is not None else data
            return _CollectStreams.apply(link, group, ranks, index, m, transfers, out_meta, *(outs if is_last else tokens))
        y = torch.cat(outs, dim=0) if is_last else torch.zeros_like(data)
        return _BroadcastFromLast.apply(y, ranks[-1], group, is_last, transfers, *tokens)


def _share_meta(out_meta, src: int, group, in_meta):
    """Shape / dtype of one output micro-batch on every rank.  Stages map ``[b, ...] -> [b, ...]``
    of the same shape in every use here, so the input's description is the output's; the last
    stage checks that."""
    del src, group
    if out_meta is not None and (tuple(out_meta[0]) != tuple(in_meta[0]) or out_meta[1] != in_meta[1]):
        raise ValueError(f"the stream schedule needs stages that keep shape and dtype: {in_meta[:2]} -> {out_meta[:2]}")
    return in_meta


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
