"""Repeat: one layer applied ``num_layers`` times with parameters stacked on a leading dim.

Parity target: ``Repeat`` in the reference (axlearn/common/repeat.py:89-223): child ``layer``,
parameter specs gain a leading ``num_layers`` dim with mesh axis ``None`` (:142-147),
initialisation uses one key per layer (:154-167), and ``_run`` scans the layer over the
stacked parameters (:172-223).

Here the scan is a Python loop, which makes three B200-specific things possible:

* the next layer's storage-sharded (FSDP) parameters are gathered on a side stream while the
  current layer computes (``LayerParamGatherer``), in forward and — in reverse order — in
  backward;
* rematerialisation is done at the loop level: per layer only the carry is kept, and in
  backward the layer's parameters are *re-gathered* (never kept unsharded), the layer is
  replayed, and its gradients are reduce-scattered straight into slice ``i`` of the stacked
  gradient buffer (``.grad`` of the stacked leaf);
* gradients of stacked leaves are written slice-wise by side effect, so no ``[L, ...]``
  zero-padded gradient is ever materialised per layer.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, Optional

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import (
    BaseLayer,
    ParameterSpec,
    _flatten_tensors,
    no_remat,
)
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.module import (
    current_context,
    new_output_collection,
    nowrap,
    set_current_context,
)
from axlearn_b200.common.utils import VDict, flatten_items, tree_map, unflatten_items
from axlearn_b200.parallel import fsdp
from axlearn_b200.parallel.mesh import current_mesh

Tensor = torch.Tensor


def _is_spec(x):
    return isinstance(x, ParameterSpec)


class _LayerCall(torch.autograd.Function):
    """Runs layer ``i`` of a Repeat.

    ``tensors`` = carry/x tensor leaves followed by the *stacked* parameter leaves.  With
    ``remat`` only these are kept and the layer is replayed in backward; without it the
    layer's autograd graph is built once (inside an inner graph rooted at the gathered
    parameters) and kept.  Either way parameter gradients leave through
    ``gatherer.scatter_grads`` into ``stacked.grad[i]``; the Function returns None for them.
    """

    @staticmethod
    def forward(ctx, run, gatherer, i, n_inputs, remat, *tensors):  # pylint: disable=arguments-differ
        # `remat`: False (keep the graph), True (keep the inputs only) or a remat.RematPolicy
        # (keep the inputs and what the policy names; the replay skips what was kept).
        from axlearn_b200.common import remat as remat_lib

        ctx.stash = remat_lib.LayerStash(remat) if isinstance(remat, remat_lib.RematPolicy) else None
        remat = bool(remat)
        ctx.run, ctx.gatherer, ctx.i, ctx.n_inputs, ctx.remat = run, gatherer, i, n_inputs, remat
        # Backward runs on an autograd worker thread, where the thread-local mesh stack is empty.
        ctx.mesh = current_mesh()
        inputs = tensors[:n_inputs]
        ctx.needs = [t.requires_grad for t in inputs]
        ctx.param_needs = [t.requires_grad for t in tensors[n_inputs:]]
        params = gatherer.get(i)
        gatherer.prefetch(i + 1)
        if remat:
            ctx.save_for_backward(*inputs)
            with torch.no_grad(), remat_lib.recording(ctx.stash):
                outs = run(inputs, params, first_pass=True)
            return tuple(outs)
        # No remat: build and keep an inner graph.
        with torch.enable_grad():
            in_d = [t.detach().requires_grad_(n) if t.is_floating_point() else t for t, n in zip(inputs, ctx.needs)]
            p_d = [p.detach().requires_grad_(n) for p, n in zip(params, ctx.param_needs)]
            outs = run(in_d, p_d, first_pass=True)
        ctx.inner = (in_d, p_d, outs)
        return tuple(o.detach() for o in outs)

    @staticmethod
    def backward(ctx, *grads):  # pylint: disable=arguments-differ
        if ctx.mesh is not None and current_mesh() is not ctx.mesh:
            with ctx.mesh:
                return _LayerCall._backward(ctx, *grads)
        return _LayerCall._backward(ctx, *grads)

    @staticmethod
    def _backward(ctx, *grads):
        gatherer, i = ctx.gatherer, ctx.i
        if ctx.remat:
            inputs = ctx.saved_tensors
            params = gatherer.get(i)
            gatherer.prefetch(i - 1)
            from axlearn_b200.common import remat as remat_lib

            with torch.enable_grad(), remat_lib.replaying(ctx.stash):
                in_d = [t.detach().requires_grad_(n) if t.is_floating_point() else t.detach() for t, n in zip(inputs, ctx.needs)]
                p_d = [p.detach().requires_grad_(n) for p, n in zip(params, ctx.param_needs)]
                outs = ctx.run(in_d, p_d, first_pass=False)
            if ctx.stash is not None:
                ctx.stash.clear()
        else:
            in_d, p_d, outs = ctx.inner
            ctx.inner = None
        pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        gatherer.scatter_grads(i, [p.grad for p in p_d])
        in_grads = tuple(
            (t.grad if n and t.is_floating_point() else None) for t, n in zip(in_d, ctx.needs)
        )
        return (None, None, None, None, None) + in_grads + (None,) * len(p_d)


class Repeat(BaseLayer):
    """Applies ``layer`` ``num_layers`` times; see the module docstring."""

    @config_class
    class Config(BaseLayer.Config):
        layer: Required[InstantiableConfig] = REQUIRED
        num_layers: Required[int] = REQUIRED
        # Paths (regex on "summaries/..." / "module_outputs/...") to drop per iteration.
        drop_output: Optional[Callable[[str], bool]] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("layer", cfg.layer)
        self._gatherer_cache: dict[int, fsdp.LayerParamGatherer] = {}

    # ------------------------------------------------------------------ parameters
    @nowrap
    def create_parameter_specs_recursively(self):
        n = self._config.num_layers

        def stack(spec: ParameterSpec) -> ParameterSpec:
            return dataclasses.replace(
                spec,
                shape=(n,) + tuple(spec.shape),
                mesh_axes=None if spec.mesh_axes is None else (None,) + tuple(spec.mesh_axes),
                fan_axes=_shift_fan_axes(spec.fan_axes),
            )

        inner = self.layer.create_parameter_specs_recursively()
        return {"layer": VDict(tree_map(stack, inner, is_leaf=_is_spec))}

    @nowrap
    def initialize_parameters_recursively(self, prng_key, *, prebuilt=None, device=None):
        n = self._config.num_layers
        pre = prebuilt.get("layer") if isinstance(prebuilt, dict) else None
        if pre is not None and all(isinstance(v, torch.Tensor) for _, v in flatten_items(pre)) and flatten_items(pre):
            return {"layer": VDict(pre)}
        # The split mirrors BaseLayer (one key per child; Repeat has the single child
        # "layer"), then one key per repetition.
        (child_key,) = prng.split(prng_key, 1)
        keys = prng.split(child_key, n)
        stacked: Optional[dict] = None
        for i, k in enumerate(keys):
            layer_i = self.layer.initialize_parameters_recursively(k, device=device)
            flat = flatten_items(layer_i)
            if stacked is None:
                stacked = {p: torch.empty((n,) + tuple(t.shape), dtype=t.dtype, device=t.device) for p, t in flat}
            for p, t in flat:
                stacked[p][i].copy_(t)
            del layer_i, flat
        return {"layer": VDict(unflatten_items(list((stacked or {}).items())))}

    # ------------------------------------------------------------------ execution
    def _gatherer(self, stacked_params: Any, *, remat: bool = False):
        leaves = [t for _, t in flatten_items(stacked_params)]
        key = hash(tuple(id(t) for t in leaves)) ^ int(remat)
        g = self._gatherer_cache.get(key)
        if g is None:
            mesh = current_mesh()
            specs = self.layer.create_parameter_specs_recursively()
            plans = tree_map(lambda s: fsdp.LeafPlan(mesh, s.mesh_axes), specs, is_leaf=_is_spec)
            from axlearn_b200.parallel import fsdp_fused

            plan_list = [p for _, p in flatten_items(plans, is_leaf=lambda x: isinstance(x, fsdp.LeafPlan))]
            # The fused path shares one gather buffer per leaf across layers, so it needs the
            # layer to be replayed (remat) rather than kept for backward.
            if remat and leaves and fsdp_fused.supported(leaves, plan_list):
                g = fsdp_fused.FusedLayerGatherer(stacked_params, plans, self._config.num_layers)
                fsdp_fused.register(g)
            else:
                g = fsdp.LayerParamGatherer(stacked_params, plans, self._config.num_layers)
            self._gatherer_cache[key] = g
        return g

    def _run(self, fn: Callable, *, carry: Any, xs: Any = None, collect: bool = False):
        """``carry, y_i = fn(carry, x_i, layer)`` for each repetition.

        Returns ``(carry, ys)`` where ``ys`` is the per-layer outputs stacked on a new leading
        dim when ``collect`` (else None).
        """
        cfg = self._config
        ctx = current_context()
        stacked_params = ctx.state.get("layer", {}) if isinstance(ctx.state, dict) else {}
        param_items = flatten_items(stacked_params)
        param_paths = [p for p, _ in param_items]
        param_leaves = [t for _, t in param_items]
        layer_cfg = cfg.layer
        remat_spec = getattr(layer_cfg, "remat_spec", None)
        training = ctx.is_training and torch.is_grad_enabled()
        use_remat = bool(training and remat_spec is not None and not remat_spec.saves_everything())
        # A selective policy (names to keep / offload) rides along in place of the plain flag.
        remat_arg = (remat_spec.selective_policy() or True) if use_remat else False
        gatherer = self._gatherer(stacked_params, remat=use_remat or not training)
        needs_param_grads = training and any(t.requires_grad for t in param_leaves)
        via_function = needs_param_grads and (use_remat or gatherer.sharded or True)

        ys = []
        state_updates: list = []     # per-layer non-gradient updates (e.g. batch-norm statistics)
        gatherer.prefetch(0)
        for i in range(cfg.num_layers):
            x_i = None if xs is None else tree_map(lambda t, i=i: t[i], xs)
            key_i = None if ctx.prng_key is None else prng.fold_in(ctx.prng_key, i)
            live_oc = new_output_collection()
            out_box: dict[str, Any] = {}
            in_tensors, rebuild_in = _flatten_tensors({"carry": carry, "x": x_i})

            def run(inputs, params, *, first_pass, i=i, key_i=key_i, live_oc=live_oc,
                    rebuild_in=rebuild_in, out_box=out_box):
                tree = rebuild_in(list(inputs))
                state_i = unflatten_items(list(zip(param_paths, params))) if param_paths else {}
                oc = live_oc if first_pass else new_output_collection()
                iter_ctx = dataclasses.replace(
                    ctx, state={"layer": state_i}, prng_key=key_i, output_collection=oc
                )
                with set_current_context(iter_ctx, require_parent=False), no_remat():
                    out = fn(tree["carry"], tree["x"], self.layer)
                out_tensors, rebuild_out = _flatten_tensors(out)
                if first_pass:
                    out_box["rebuild"] = rebuild_out
                return out_tensors

            if via_function:
                outs = _LayerCall.apply(
                    run, gatherer, i, len(in_tensors), remat_arg, *in_tensors, *param_leaves
                )
            else:
                params = gatherer.get(i)
                gatherer.prefetch(i + 1)
                outs = run(in_tensors, params, first_pass=True)
            carry, y_i = out_box["rebuild"](list(outs))
            if collect:
                ys.append(y_i)
            # File this iteration's side outputs under layer{i}.
            if cfg.drop_output is not None:
                from axlearn_b200.common.module import _prune_paths

                _prune_paths(live_oc.summaries, cfg.drop_output)
                _prune_paths(live_oc.module_outputs, cfg.drop_output)
            child = ctx.output_collection.get_or_add_child(f"layer{i}")
            child.summaries.update(live_oc.summaries.get("layer", {}))
            child.module_outputs.update(live_oc.module_outputs.get("layer", {}))
            updates_i = live_oc.state_updates.get("layer", {})
            if flatten_items(updates_i):
                state_updates.append(updates_i)
        if state_updates:
            # Every repetition updates the same parameters: the new values of the stacked
            # parameters are the per-layer values stacked on the layer dim.
            if len(state_updates) != cfg.num_layers:
                raise NotImplementedError("state updates must come from every repetition of a Repeat")
            stacked = tree_map(lambda *ts: torch.stack([t.detach() for t in ts], dim=0), *state_updates)
            ctx.output_collection.state_updates.setdefault("layer", {})
            _merge_dicts(ctx.output_collection.state_updates["layer"], stacked)
        stacked_ys = None
        if collect and ys:
            if any(t is not None for t in ys) and _flatten_tensors(ys[0])[0]:
                stacked_ys = tree_map(lambda *ts: torch.stack(ts, dim=0), *ys)
            else:
                stacked_ys = ys
        return carry, stacked_ys

    def forward(self, carry, **kwargs):
        def body(c, _x, layer):
            return layer(c, **kwargs), None

        out, _ = self._run(body, carry=carry)
        return out


def _merge_dicts(dst: dict, src: dict) -> None:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _merge_dicts(dst[k], v)
        else:
            dst[k] = v


def _shift_fan_axes(fan_axes):
    """Fan axes of a stacked parameter: the new leading dim is a batch axis; non-negative
    axes move right by one."""
    if fan_axes is None:
        return None
    from axlearn_b200.common.param_init import FanAxes

    def shift(a):
        if isinstance(a, int):
            return a + 1 if a >= 0 else a
        return tuple(shift(x) for x in a)

    batch = shift(fan_axes.batch_axis)
    batch = (batch,) if isinstance(batch, int) else tuple(batch)
    return FanAxes(in_axis=shift(fan_axes.in_axis), out_axis=shift(fan_axes.out_axis), batch_axis=(0,) + batch)
