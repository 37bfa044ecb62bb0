"""Learner: owns the optimizer, decides which parameters update how, applies updates.

Parity targets in the reference (axlearn/common/learner.py): ``UpdateType`` (:62-94),
``Learner`` (:156) with ``create_state_partition_specs`` (:200-228), ``init`` (:230-240),
``update`` (:265-357), ``forward_and_backward`` (:359-374), update rules (:242-260),
``CompositeLearner`` (:404-627) and gradient splitting (:630-681).

State layout: ``{"optimizer": <transformation state>, ["ema": <ParamEmaState>]}``.

Mixed precision: the trainer keeps fp32 master parameters in its state and, when the step
dtype differs, a persistent low-precision *shadow* of each trainable parameter that the model
actually reads.  Gradients arrive on the shadows (in the step dtype); the update writes the
master and refreshes the shadow in the same pass — on the fused path inside the AdamW kernel —
so no separate "cast params" pass over the model exists.
"""

from __future__ import annotations

import enum
import re
from typing import Any, Callable, Optional, Sequence

import torch

from axlearn_b200.common import optimizers as opt_lib
from axlearn_b200.common.base_layer import ParameterSpec
from axlearn_b200.common.config import (
    REQUIRED,
    InstantiableConfig,
    Required,
    config_class,
    config_for_function,
)
from axlearn_b200.common.module import Module
from axlearn_b200.common.optimizer_base import OptParam, PartitionedGradientTransformation
from axlearn_b200.common.utils import (
    TensorSpec,
    flatten_items,
    match_regex_rules,
    tree_map,
    tree_paths,
    unflatten_items,
)
from axlearn_b200.parallel import fsdp, grad_sync

Tensor = torch.Tensor
_is_spec = lambda x: isinstance(x, TensorSpec)


class UpdateType(enum.Enum):
    """How a parameter may change during training."""

    NO_UPDATE = "no_update"  # Frozen.
    OPTIMIZERS = "optimizers"  # Only through the optimizer.
    STATE_UPDATES = "state_updates"  # Only through add_state_update (e.g. BN statistics).
    ALL_UPDATES = "all_updates"


def should_update_with_optimizers(t: UpdateType) -> bool:
    return t in (UpdateType.OPTIMIZERS, UpdateType.ALL_UPDATES)


def should_apply_state_updates(t: UpdateType) -> bool:
    return t in (UpdateType.STATE_UPDATES, UpdateType.ALL_UPDATES)


class BaseLearner(Module):
    @config_class
    class Config(Module.Config):
        pass

    def init(self, model_params: Any) -> Any:
        raise NotImplementedError(type(self))

    def create_state_partition_specs(self, model_param_specs: Any) -> Any:
        raise NotImplementedError(type(self))


class Learner(BaseLearner):
    @config_class
    class Config(BaseLearner.Config):
        optimizer: Required[InstantiableConfig] = REQUIRED
        # [(regex on param path, UpdateType)]; first full match wins; default ALL_UPDATES.
        update_rules: Sequence[tuple[str, UpdateType]] = []
        # param_ema config (set ``ema.decay`` to enable).
        ema: InstantiableConfig = config_for_function(opt_lib.param_ema)
        enable_per_variable_summaries: bool = False
        # Use the fused multi-tensor kernel when the optimizer provides a closed form.
        allow_fused_update: bool = True

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self.optimizer: PartitionedGradientTransformation = cfg.optimizer.instantiate()
        self.ema: Optional[PartitionedGradientTransformation] = (
            cfg.ema.instantiate() if cfg.ema.decay is not None else None
        )
        self._allow_contextless = True

    # ------------------------------------------------------------------ rules
    def update_types(self, tree: Any) -> Any:
        rules = self._config.update_rules
        return tree_map(
            lambda path: match_regex_rules(path, rules=rules, default_value=UpdateType.ALL_UPDATES),
            tree_paths(tree, is_leaf=lambda x: isinstance(x, (TensorSpec, OptParam))),
        )

    def should_update_with_optimizers(self, tree: Any) -> Any:
        return tree_map(should_update_with_optimizers, self.update_types(tree))

    def _trainable(self, tree: Any) -> Any:
        """Sub-tree of leaves handled by the optimizer (others pruned)."""
        keep = dict(flatten_items(self.should_update_with_optimizers(tree)))
        items = [(p, v) for p, v in flatten_items(tree, is_leaf=lambda x: isinstance(x, (TensorSpec, OptParam))) if keep.get(p, True)]
        return unflatten_items(items)

    # ------------------------------------------------------------------ state
    def create_state_partition_specs(self, model_param_specs: Any) -> Any:
        specs = self._trainable(model_param_specs)
        out = {"optimizer": self.optimizer.partition(specs)}
        if self.ema is not None:
            out["ema"] = self.ema.partition(model_param_specs)
        return out

    def init(self, model_params: Any) -> Any:
        """``model_params``: tree of OptParam."""
        out = {"optimizer": self.optimizer.init(self._trainable(model_params))}
        if self.ema is not None:
            out["ema"] = self.ema.init(model_params)
        return out

    # ------------------------------------------------------------------ update
    def update(
        self,
        *,
        model_params: Any,
        gradients: Any,
        state: Any,
        param_specs: Any,
        state_updates: Optional[dict] = None,
        shadows: Optional[Any] = None,
    ) -> Any:
        """Applies one optimizer step **in place** on ``model_params`` (fp32 masters) and
        refreshes ``shadows``; returns the new learner state.

        ``gradients`` mirrors ``model_params`` with ``None`` for parameters without gradient.
        """
        cfg = self._config
        flat_params = dict(flatten_items(model_params))
        flat_specs = dict(flatten_items(param_specs, is_leaf=_is_spec))
        flat_grads = dict(flatten_items(gradients, is_leaf=lambda x: x is None or isinstance(x, torch.Tensor)))
        flat_shadows = dict(flatten_items(shadows)) if shadows is not None else {}
        types = dict(flatten_items(self.update_types(param_specs)))
        train_paths = [p for p in flat_params if should_update_with_optimizers(types.get(p, UpdateType.ALL_UPDATES))
                       and flat_grads.get(p) is not None]
        opt_params = unflatten_items([
            (p, OptParam(flat_params[p], getattr(flat_specs.get(p), "factorization", None),
                         getattr(flat_specs.get(p), "weight_decay_scale", None)))
            for p in flat_params if should_update_with_optimizers(types.get(p, UpdateType.ALL_UPDATES))
        ])
        grads_tree = unflatten_items([
            (p, flat_grads.get(p)) for p in flat_params
            if should_update_with_optimizers(types.get(p, UpdateType.ALL_UPDATES))
        ])
        specs_tree = unflatten_items([(p, flat_specs[p]) for p in flat_params
                                      if p in flat_specs and should_update_with_optimizers(types.get(p, UpdateType.ALL_UPDATES))])
        new_state = dict(state)
        with torch.no_grad(), opt_lib.param_specs_scope(specs_tree):
            fused = self.optimizer.fused if cfg.allow_fused_update else None
            if fused is not None and not cfg.enable_per_variable_summaries:
                new_state["optimizer"] = _fused_update(
                    fused, grads=grads_tree, state=state["optimizer"], params=opt_params,
                    specs=specs_tree, shadows=flat_shadows, add_summary=self._maybe_summary)
            else:
                grads32 = tree_map(lambda g: None if g is None else g.float(), grads_tree,
                                   is_leaf=lambda x: x is None or isinstance(x, torch.Tensor))
                updates, new_state["optimizer"] = self.optimizer.update(grads32, state["optimizer"], opt_params)
                flat_updates = dict(flatten_items(updates, is_leaf=lambda x: x is None or isinstance(x, torch.Tensor)))
                for p in train_paths:
                    u = flat_updates.get(p)
                    if u is None:
                        continue
                    flat_params[p].add_(u.to(flat_params[p].dtype))
                    if cfg.enable_per_variable_summaries:
                        self._maybe_summary(f"param_rms/{p}", flat_params[p].float().pow(2).mean().sqrt())
                        self._maybe_summary(f"grad_rms/{p}", flat_grads[p].float().pow(2).mean().sqrt())
                for p in train_paths:
                    sh = flat_shadows.get(p)
                    if sh is not None and sh is not flat_params[p]:
                        sh.copy_(flat_params[p])
            # Non-gradient state updates (e.g. batch-norm statistics).
            for p, v in flatten_items(state_updates or {}):
                if p in flat_params and should_apply_state_updates(types.get(p, UpdateType.ALL_UPDATES)):
                    flat_params[p].copy_(v.to(flat_params[p].dtype))
                    sh = flat_shadows.get(p)
                    if sh is not None and sh is not flat_params[p]:
                        sh.copy_(flat_params[p])
            if self.ema is not None:
                all_params = tree_map(lambda t: OptParam(t, None, None), model_params)
                _, new_state["ema"] = self.ema.update(None, state["ema"], all_params)
        return new_state

    def _maybe_summary(self, name: str, value: Any) -> None:
        from axlearn_b200.common.module import current_context

        ctx = current_context()
        if ctx is not None:
            ctx.add_summary(name, value)


def _fused_update(fused: opt_lib.FusedSpec, *, grads, state, params, specs, shadows, add_summary):
    """One multi-tensor AdamW step over all trainable leaves, using and updating the same
    state tree as the generic chain."""
    from axlearn_b200.ops import optim

    adam_state, counters, _ = fused.locate(state)
    flat_g = flatten_items(grads, is_leaf=lambda x: x is None or isinstance(x, torch.Tensor))
    flat_p = dict(flatten_items(params, is_leaf=lambda x: isinstance(x, OptParam)))
    flat_m = dict(flatten_items(adam_state.mu))
    flat_v = dict(flatten_items(adam_state.nu))
    scales = dict(flatten_items(opt_lib._weight_decay_scales(params, fused.per_param_scale)))  # pylint: disable=protected-access
    live = [(p, g) for p, g in flat_g if g is not None]
    grad_scale = 1.0
    if fused.clip_max_norm is not None:
        g_norm = opt_lib.global_norm(unflatten_items(live), specs=specs)
        add_summary("gradient_norm", g_norm)
        gn = g_norm  # Stays on device: the kernel reads the scale from memory.
        grad_scale = torch.clamp(fused.clip_max_norm / (gn + fused.clip_eps), max=1.0)
        add_summary("gradient_scale", grad_scale)
    count = (adam_state.count + 1).to(torch.int32)
    t = int(count)
    lr = fused.learning_rate(t)
    s = fused.update_schedule(t)
    add_summary("lr/schedule_step" if fused.decoupled else "schedule_step", count)
    add_summary("lr/schedule_scale" if fused.decoupled else "schedule_scale", lr)
    if fused.decoupled:
        add_summary("update/schedule_step", count)
        add_summary("update/schedule_scale", s)
        step_lr, step_wd = s * lr, s * fused.weight_decay
    else:
        step_lr, step_wd = lr, lr * fused.weight_decay
    optim.multi_tensor_adamw(
        params=[flat_p[p].value for p, _ in live],
        grads=[g for _, g in live],
        mus=[flat_m[p] for p, _ in live],
        nus=[flat_v[p] for p, _ in live],
        shadows=[shadows.get(p) for p, _ in live],
        wd_scales=[float(scales[p]) for p, _ in live],
        step=t, lr=step_lr, weight_decay=step_wd, b1=fused.b1, b2=fused.b2, eps=fused.eps,
        grad_scale=grad_scale,
    )
    # Rebuild the state with incremented counters (same structure as the generic chain).
    new_adam = opt_lib.ScaleByAdamState(count, adam_state.mu, adam_state.nu)
    return _rebuild_fused_state(state, fused, new_adam, count)


def _rebuild_fused_state(state, fused: opt_lib.FusedSpec, new_adam, count):
    adam_state, counters, chain_index = fused.locate(state)

    def rebuild_inner(inner_state):
        inner = list(inner_state)
        inner[0] = new_adam
        for idx, st in counters:
            if getattr(st, "count", None) is not None:
                inner[idx] = type(st)(count.clone())
        return tuple(inner)

    if chain_index is None:
        return rebuild_inner(state)
    outer = list(state)
    outer[chain_index] = rebuild_inner(state[chain_index])
    return tuple(outer)


class CompositeLearner(BaseLearner):
    """Routes parameters to sub-learners by regex on the parameter path."""

    @config_class
    class Config(BaseLearner.Config):
        # [(regex, learner name)]; every parameter must match exactly one rule.
        rules: Required[Sequence[tuple[str, str]]] = REQUIRED
        learners: Required[dict[str, InstantiableConfig]] = REQUIRED
        ema: InstantiableConfig = config_for_function(opt_lib.param_ema)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._learners = {}
        for name, lcfg in cfg.learners.items():
            if lcfg.ema.decay is not None:
                raise ValueError("sub-learner ema is not supported; set ema on the CompositeLearner")
            self._learners[name] = self._add_child(name, lcfg)
        self.ema = cfg.ema.instantiate() if cfg.ema.decay is not None else None
        self._allow_contextless = True

    def _owner(self, path: str) -> str:
        name = match_regex_rules(path, rules=self._config.rules, default_value=None)
        if name is None:
            raise ValueError(f"{path} matches no learner rule")
        if name not in self._learners:
            raise ValueError(f"rule maps {path} to unknown learner {name}")
        return name

    def _split(self, tree: Any, is_leaf=None) -> dict[str, Any]:
        parts: dict[str, list] = {n: [] for n in self._learners}
        for p, v in flatten_items(tree, is_leaf=is_leaf):
            parts[self._owner(p)].append((p, v))
        return {n: unflatten_items(items) for n, items in parts.items()}

    def create_state_partition_specs(self, model_param_specs: Any) -> Any:
        parts = self._split(model_param_specs, is_leaf=_is_spec)
        out = {n: self._learners[n].create_state_partition_specs(parts[n]) for n in self._learners}
        if self.ema is not None:
            out["ema"] = self.ema.partition(model_param_specs)
        return out

    def init(self, model_params: Any) -> Any:
        parts = self._split(model_params, is_leaf=lambda x: isinstance(x, OptParam))
        out = {n: self._learners[n].init(parts[n]) for n in self._learners}
        if self.ema is not None:
            out["ema"] = self.ema.init(model_params)
        return out

    def update(self, *, model_params, gradients, state, param_specs, state_updates=None, shadows=None):
        p_parts = self._split(model_params)
        g_parts = self._split(gradients, is_leaf=lambda x: x is None or isinstance(x, torch.Tensor))
        s_parts = self._split(param_specs, is_leaf=_is_spec)
        sh_parts = self._split(shadows) if shadows is not None else {n: None for n in self._learners}
        su_parts = self._split(state_updates or {})
        new_state = dict(state)
        for n, learner in self._learners.items():
            new_state[n] = learner.update(
                model_params=p_parts[n], gradients=g_parts[n], state=state[n], param_specs=s_parts[n],
                state_updates=su_parts.get(n), shadows=sh_parts[n])
        if self.ema is not None:
            with torch.no_grad():
                all_params = tree_map(lambda t: OptParam(t, None, None), model_params)
                _, new_state["ema"] = self.ema.update(None, state["ema"], all_params)
        return new_state

    def update_types(self, tree: Any) -> Any:
        merged: list = []
        parts = self._split(tree, is_leaf=lambda x: isinstance(x, (TensorSpec, OptParam)))
        for n, learner in self._learners.items():
            merged.extend(flatten_items(learner.update_types(parts[n])))
        return unflatten_items(merged)
