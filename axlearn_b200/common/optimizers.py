"""Optimizers as composable gradient transformations.

Parity targets in the reference (axlearn/common/optimizers.py): ``chain`` / ``named_chain``
(:81-110), ``scale`` / ``scale_by_schedule`` (:221-268), ``per_param_scale_by_path`` (:287),
``scale_by_trust_ratio`` (:348), ``scale_update_per_param`` (:467), ``add_decayed_weights``
(:552-634), ``l2_regularizer`` (:636), ``sgd_optimizer`` (:685), ``adamw_optimizer`` (:741),
``adamw_decoupled_optimizer`` (:796), ``adam_optimizer`` (:859), ``ema`` (:888),
``adafactor_optimizer`` (:1058), ``clip_by_global_norm`` (:1149),
``skip_and_clip_by_global_norm`` (:1254), ``clip_by_block_rms`` (:1509), ``param_ema`` (:1592),
``lion_optimizer`` (:1709), ``offload_optimizer`` (:2095).

State layout is the reference's: a ``chain`` keeps a tuple of sub-states, stateless links keep
``EmptyState``; Adam keeps ``ScaleByAdamState(count, mu, nu)``; schedules keep
``ScaleByScheduleState(count)`` — so checkpoint leaf names such as
``learner/optimizer/1/0/mu/<param path>`` are preserved.  Counters are int32 scalars on the
host (schedules are host functions); every step is 1-based.

Two execution paths share that state:

* the generic path evaluates each link as tree-wide tensor ops (any composition, CPU or GPU);
* transformations that can be written in closed form carry ``fused`` — the learner then runs
  ONE multi-tensor kernel per step over (master param, grad, mu, nu [, bf16 shadow]) with the
  global-norm clip scale folded in.  ``chain(clip_by_global_norm, adamw_decoupled_optimizer)``
  (the Fuji recipe) and plain ``adamw_*`` qualify.
"""

from __future__ import annotations

import dataclasses
import math
import re
from typing import Any, Callable, NamedTuple, Optional, Sequence, Union

import torch

from axlearn_b200.common import schedule
from axlearn_b200.common.config import maybe_instantiate
from axlearn_b200.common.module import current_context
from axlearn_b200.common.optimizer_base import (
    EmptyState,
    OptParam,
    OptStateSpec,
    PartitionedGradientTransformation,
)
from axlearn_b200.common.utils import (
    PartitionSpec,
    TensorSpec,
    flatten_items,
    match_regex_rules,
    tree_map,
    tree_paths,
)

Tensor = torch.Tensor
_is_opt_param = lambda x: isinstance(x, OptParam)
_is_spec = lambda x: isinstance(x, TensorSpec)


def _count0() -> Tensor:
    return torch.zeros((), dtype=torch.int32)


def _inc(count: Tensor) -> Tensor:
    return (count + 1).to(torch.int32)


def _count_spec() -> OptStateSpec:
    return OptStateSpec(shape=(), dtype=torch.int32, mesh_axes=PartitionSpec())


def _summary(name: str, value: Any) -> None:
    ctx = current_context()
    if ctx is not None:
        ctx.add_summary(name, value)


def _map_updates(fn: Callable, updates: Any, *rest: Any) -> Any:
    """tree_map over updates that leaves ``None`` updates alone."""
    return tree_map(lambda u, *r: None if u is None else fn(u, *r), updates, *rest,
                    is_leaf=lambda x: x is None or isinstance(x, (torch.Tensor, OptParam)))


def _values(params: Any) -> Any:
    return tree_map(lambda p: p.value, params, is_leaf=_is_opt_param)


# ------------------------------------------------------------------------------------------
# Composition.
# ------------------------------------------------------------------------------------------


def chain(*args: Any) -> PartitionedGradientTransformation:
    """Applies transformations in order; state is the tuple of their states."""
    txs = [maybe_instantiate(a) for a in args]

    def init(params):
        return tuple(t.init(params) for t in txs)

    def update(updates, state, params):
        new = []
        for t, s in zip(txs, state):
            updates, s2 = t.update(updates, s, params)
            new.append(s2)
        return updates, tuple(new)

    def partition(specs):
        return tuple(t.partition(specs) for t in txs)

    return PartitionedGradientTransformation(init, update, partition, fused=_fuse_chain(txs))


def named_chain(**kwargs: Any) -> PartitionedGradientTransformation:
    """Like ``chain`` with a dict state keyed by the given names."""
    txs = {k: maybe_instantiate(v) for k, v in kwargs.items()}

    def init(params):
        return {k: t.init(params) for k, t in txs.items()}

    def update(updates, state, params):
        new = {}
        for k, t in txs.items():
            updates, new[k] = t.update(updates, state[k], params)
        return updates, new

    def partition(specs):
        return {k: t.partition(specs) for k, t in txs.items()}

    return PartitionedGradientTransformation(init, update, partition)


def with_partition_fn(init, update, partition) -> PartitionedGradientTransformation:
    return PartitionedGradientTransformation(init, update, partition)


def _stateless(update_fn: Callable) -> PartitionedGradientTransformation:
    return PartitionedGradientTransformation(
        init=lambda params: EmptyState(),
        update=lambda u, s, p: (update_fn(u, p), s),
        partition=lambda specs: EmptyState(),
    )


def replace_with_updates() -> PartitionedGradientTransformation:
    """The parameter's new value is its "gradient" (reference: axlearn/common/optimizers.py:202).

    The learner adds the update to the parameter, so the update is ``gradient - value``.
    """

    def fn(updates, params):
        if params is None:
            raise ValueError("replace_with_updates needs the parameters")
        return _map_updates(lambda u, p: u - p.value.to(u.dtype), updates, params)

    return _stateless(fn)


def scale(step_size: float) -> PartitionedGradientTransformation:
    return _stateless(lambda u, p: _map_updates(lambda g: g * step_size, u))


class ScaleByScheduleState(NamedTuple):
    count: Tensor


def scale_by_schedule(step_size_fn: schedule.Schedule, *, name: Optional[str] = None, flip_sign: bool = False):
    """Multiplies updates by ``schedule(count + 1)`` (1-based)."""
    fn = schedule.as_schedule_fn(step_size_fn)
    prefix = "" if name is None else f"{name}/"

    def update(updates, state, params=None):
        count = _inc(state.count)
        s = fn(int(count))
        _summary(prefix + "schedule_step", count)
        _summary(prefix + "schedule_scale", s)
        s = -s if flip_sign else s
        return _map_updates(lambda g: g * s, updates), ScaleByScheduleState(count)

    return PartitionedGradientTransformation(
        init=lambda params: ScaleByScheduleState(_count0()),
        update=update,
        partition=lambda specs: ScaleByScheduleState(_count_spec()),
    )


def per_param_scale_by_path(*, scale_by_path: Sequence[tuple[str, float]], description: str,
                            default_scale: float = 1.0) -> Callable[[Any], Any]:
    """Returns ``params -> tree of floats`` chosen by the first regex matching each path."""

    def fn(params):
        return tree_map(
            lambda path: match_regex_rules(path, rules=scale_by_path, default_value=default_scale),
            tree_paths(params, is_leaf=_is_opt_param),
        )

    fn.description = description
    return fn


def _weight_decay_scales(params: Any, per_param_scale: Optional[Callable]) -> Any:
    per_param_scale = maybe_instantiate(per_param_scale)     # a config_for_function(...) is accepted too
    scales = per_param_scale(params) if per_param_scale is not None else tree_map(lambda p: 1.0, params, is_leaf=_is_opt_param)
    return tree_map(
        lambda p, s: s if p.weight_decay_scale is None else p.weight_decay_scale,
        params, scales, is_leaf=_is_opt_param)


def scale_update_per_param(per_param_scale: Callable[[Any], Any]) -> PartitionedGradientTransformation:
    per_param_scale = maybe_instantiate(per_param_scale)

    def fn(updates, params):
        scales = per_param_scale(params)
        return _map_updates(lambda g, s: g * s, updates, scales)

    return _stateless(fn)


class AddDecayedWeightsState(NamedTuple):
    count: Optional[Tensor]


def add_decayed_weights(weight_decay: float, *, learning_rate_exponent: Optional[float] = None,
                        learning_rate: Optional[schedule.Schedule] = None,
                        per_param_scale: Optional[Callable] = None) -> PartitionedGradientTransformation:
    """``u += weight_decay * lr**exponent * scale_p * p``."""
    lr_fn = schedule.as_schedule_fn(learning_rate) if learning_rate_exponent is not None else None

    def update(updates, state, params):
        if params is None:
            raise ValueError("add_decayed_weights requires params")
        if lr_fn is None:
            lr_scale, new_state = 1.0, state
        else:
            count = _inc(state.count)
            lr_scale, new_state = lr_fn(int(count)) ** learning_rate_exponent, AddDecayedWeightsState(count)
        scales = _weight_decay_scales(params, per_param_scale)
        out = _map_updates(
            lambda g, p, s: g + (weight_decay * lr_scale * s) * p.value.to(g.dtype), updates, params, scales)
        return out, new_state

    return PartitionedGradientTransformation(
        init=lambda params: AddDecayedWeightsState(None if lr_fn is None else _count0()),
        update=update,
        partition=lambda specs: AddDecayedWeightsState(None if lr_fn is None else _count_spec()),
    )


def l2_regularizer(regularizer_weight: float = 0.0, per_param_scale: Optional[Callable] = None):
    """Adds the gradient of ``0.5 * w * ||p||^2`` (coupled L2)."""
    if not regularizer_weight:
        return _stateless(lambda u, p: u)

    def fn(updates, params):
        scales = _weight_decay_scales(params, per_param_scale)
        return _map_updates(lambda g, p, s: g + regularizer_weight * s * p.value.to(g.dtype), updates, params, scales)

    return _stateless(fn)


# ------------------------------------------------------------------------------------------
# Adam family.
# ------------------------------------------------------------------------------------------


class ScaleByAdamState(NamedTuple):
    count: Tensor
    mu: Any
    nu: Any


def _copy_specs(specs: Any, dtype: Optional[torch.dtype] = None) -> Any:
    return tree_map(
        lambda s: OptStateSpec(shape=tuple(s.shape), dtype=dtype or s.dtype, mesh_axes=s.mesh_axes),
        specs, is_leaf=_is_spec)


def scale_by_adam(b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, eps_root: float = 0.0,
                  mu_dtype: Optional[torch.dtype] = None) -> PartitionedGradientTransformation:
    """``u = m_hat / (sqrt(v_hat + eps_root) + eps)`` with bias correction by ``count + 1``."""

    def init(params):
        zeros = lambda p: torch.zeros_like(p.value, dtype=mu_dtype or p.value.dtype)
        return ScaleByAdamState(
            _count0(),
            tree_map(zeros, params, is_leaf=_is_opt_param),
            tree_map(lambda p: torch.zeros_like(p.value), params, is_leaf=_is_opt_param),
        )

    def update(updates, state, params=None):
        count = _inc(state.count)
        t = int(count)

        def upd(g, m, v):
            gf = g.to(v.dtype)
            m.mul_(b1).add_(gf.to(m.dtype), alpha=1 - b1)
            v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
            mhat = m.to(v.dtype) / (1 - b1**t)
            vhat = v / (1 - b2**t)
            return mhat / (torch.sqrt(vhat + eps_root) + eps)

        out = _map_updates(upd, updates, state.mu, state.nu)
        return out, ScaleByAdamState(count, state.mu, state.nu)

    def partition(specs):
        return ScaleByAdamState(_count_spec(), _copy_specs(specs, mu_dtype), _copy_specs(specs))

    return PartitionedGradientTransformation(init, update, partition)


@dataclasses.dataclass
class FusedSpec:
    """Closed form of ``[clip] -> adam -> lr -> weight decay -> update schedule -> negate``.

    ``locate(state)`` returns the ``(adam_state, [counter states...])`` inside the owning
    transformation's state and ``rebuild`` puts updated ones back.
    """

    b1: float
    b2: float
    eps: float
    learning_rate: Callable[[int], float]
    update_schedule: Callable[[int], float]
    weight_decay: float
    per_param_scale: Optional[Callable]
    decoupled: bool  # True: p -= s*(lr*u + wd*p); False: p -= lr*(u + wd*p)
    clip_max_norm: Optional[float] = None
    clip_eps: float = 1e-8
    locate: Optional[Callable] = None


def adamw_optimizer(learning_rate: schedule.Schedule, *, b1: float, b2: float, eps: float,
                    weight_decay: float = 0.0, weight_decay_per_param_scale: Optional[Callable] = None,
                    mu_dtype: Optional[torch.dtype] = None,
                    adam_update_transformation: Optional[Any] = None) -> PartitionedGradientTransformation:
    """AdamW with weight decay scaled by the learning rate:
    ``p -= lr_t * (m_hat/(sqrt(v_hat)+eps) + wd * p)``."""
    links = [scale_by_adam(b1=b1, b2=b2, eps=eps, mu_dtype=mu_dtype)]
    if adam_update_transformation is not None:
        links.append(maybe_instantiate(adam_update_transformation))
    links += [
        add_decayed_weights(weight_decay, per_param_scale=weight_decay_per_param_scale),
        scale_by_schedule(learning_rate, flip_sign=True),
    ]
    tx = chain(*links)
    if adam_update_transformation is None:
        lr = schedule.as_schedule_fn(learning_rate)
        tx.fused = FusedSpec(
            b1=b1, b2=b2, eps=eps, learning_rate=lr, update_schedule=lambda t: 1.0,
            weight_decay=weight_decay, per_param_scale=weight_decay_per_param_scale, decoupled=False,
            locate=lambda st: (st[0], [(2, st[2])], None),
        )
        if mu_dtype is not None:
            tx.fused = None
    return tx


def adamw_decoupled_optimizer(learning_rate: float, *, b1: float, b2: float, eps: float,
                              update_schedule: schedule.Schedule, weight_decay: float = 0.0,
                              weight_decay_per_param_scale: Optional[Callable] = None,
                              mu_dtype: Optional[torch.dtype] = None,
                              adam_update_transformation: Optional[Any] = None) -> PartitionedGradientTransformation:
    """AdamW with weight decay decoupled from the learning rate:
    ``p -= s_t * (lr * m_hat/(sqrt(v_hat)+eps) + wd * scale_p * p)`` where ``s_t`` is the
    update schedule at the 1-based step."""
    links = [scale_by_adam(b1=b1, b2=b2, eps=eps, mu_dtype=mu_dtype)]
    if adam_update_transformation is not None:
        links.append(maybe_instantiate(adam_update_transformation))
    links += [
        scale_by_schedule(learning_rate, name="lr"),
        add_decayed_weights(weight_decay, per_param_scale=weight_decay_per_param_scale),
        scale_by_schedule(update_schedule, name="update"),
        scale(-1.0),
    ]
    tx = chain(*links)
    if adam_update_transformation is None and mu_dtype is None:
        tx.fused = FusedSpec(
            b1=b1, b2=b2, eps=eps, learning_rate=schedule.as_schedule_fn(learning_rate),
            update_schedule=schedule.as_schedule_fn(update_schedule), weight_decay=weight_decay,
            per_param_scale=weight_decay_per_param_scale, decoupled=True,
            locate=lambda st: (st[0], [(1, st[1]), (3, st[3])], None),
        )
    return tx


def adam_optimizer(learning_rate: schedule.Schedule, *, b1: float, b2: float, eps: float,
                   l2_regularizer_weight: float = 0.0, l2_regularizer_per_param_scale: Optional[Callable] = None,
                   mu_dtype: Optional[torch.dtype] = None) -> PartitionedGradientTransformation:
    """Adam with optional coupled L2 regularisation (added to the gradient before Adam)."""
    return chain(
        l2_regularizer(l2_regularizer_weight, l2_regularizer_per_param_scale),
        scale_by_adam(b1=b1, b2=b2, eps=eps, mu_dtype=mu_dtype),
        scale_by_schedule(learning_rate, flip_sign=True),
    )


def _fuse_chain(txs: Sequence[PartitionedGradientTransformation]) -> Optional[FusedSpec]:
    """``chain(clip_by_global_norm, <fusable adam>)`` is itself fusable."""
    if len(txs) == 2 and getattr(txs[0], "clip_spec", None) is not None and txs[1].fused is not None:
        inner = txs[1].fused
        max_norm, eps = txs[0].clip_spec

        def locate(state, inner=inner):
            adam, counters, _ = inner.locate(state[1])
            return adam, counters, 1

        return dataclasses.replace(inner, clip_max_norm=max_norm, clip_eps=eps, locate=locate)
    if len(txs) == 1 and txs[0].fused is not None:
        inner = txs[0].fused

        def locate1(state, inner=inner):
            adam, counters, _ = inner.locate(state[0])
            return adam, counters, 0

        return dataclasses.replace(inner, locate=locate1)
    return None


# ------------------------------------------------------------------------------------------
# SGD / momentum / Lion / Adafactor.
# ------------------------------------------------------------------------------------------


class TraceState(NamedTuple):
    trace: Any


def trace(decay: float, nesterov: bool = False) -> PartitionedGradientTransformation:
    def init(params):
        return TraceState(tree_map(lambda p: torch.zeros_like(p.value), params, is_leaf=_is_opt_param))

    def update(updates, state, params=None):
        def upd(g, t):
            t.mul_(decay).add_(g.to(t.dtype))
            return (g + decay * t) if nesterov else t.clone()

        return _map_updates(upd, updates, state.trace), state

    return PartitionedGradientTransformation(init, update, lambda specs: TraceState(_copy_specs(specs)))


def sgd_optimizer(learning_rate: schedule.Schedule, *, decouple_weight_decay: bool, momentum: float = 0.0,
                  weight_decay: float = 0.0, weight_decay_per_param_scale: Optional[Callable] = None):
    links = []
    if not decouple_weight_decay:
        links.append(add_decayed_weights(weight_decay, per_param_scale=weight_decay_per_param_scale))
    if momentum:
        links.append(trace(momentum))
    if decouple_weight_decay:
        links.append(add_decayed_weights(weight_decay, per_param_scale=weight_decay_per_param_scale))
    links.append(scale_by_schedule(learning_rate, flip_sign=True))
    return chain(*links)


class LionState(NamedTuple):
    count: Tensor
    mu: Any


def lion_optimizer(learning_rate: schedule.Schedule, *, b1: float = 0.9, b2: float = 0.99,
                   mu_dtype: Optional[torch.dtype] = None, weight_decay: float = 0.0,
                   multiply_by_parameter_scale: bool = False,
                   weight_decay_per_param_scale: Optional[Callable] = None):
    """Lion: ``u = sign(b1*m + (1-b1)*g)``; ``m = b2*m + (1-b2)*g``."""

    def init(params):
        return LionState(_count0(), tree_map(lambda p: torch.zeros_like(p.value, dtype=mu_dtype or p.value.dtype), params, is_leaf=_is_opt_param))

    def update(updates, state, params=None):
        def upd(g, m):
            u = torch.sign(b1 * m.to(g.dtype) + (1 - b1) * g)
            m.mul_(b2).add_(g.to(m.dtype), alpha=1 - b2)
            return u

        return _map_updates(upd, updates, state.mu), LionState(_inc(state.count), state.mu)

    lion = PartitionedGradientTransformation(init, update, lambda specs: LionState(_count_spec(), _copy_specs(specs, mu_dtype)))
    links = [lion]
    if multiply_by_parameter_scale:
        links.append(scale_by_param_block_rms())
    links += [add_decayed_weights(weight_decay, per_param_scale=weight_decay_per_param_scale),
              scale_by_schedule(learning_rate, flip_sign=True)]
    return chain(*links)


class AdastarState(NamedTuple):
    count: Tensor
    gradient_ema: Any           # None when gradient_ema_decay is None
    gradient_square_ema: Any
    update_ema: Any             # None when update_ema_decay is None


def adastar_optimizer(learning_rate: float, *, gradient_ema_decay: Optional[float], gradient_ema_debias: bool,
                      gradient_square_ema_decay: float, gradient_square_ema_debias: bool, eps: float,
                      eps_square: float, raw_update_clipping_threshold: Optional[float],
                      update_ema_decay: Optional[float], update_ema_debias: bool,
                      adam_update_transformation: Optional[Any] = None, weight_decay: float = 0.0,
                      weight_decay_per_param_scale: Optional[Callable] = None,
                      update_schedule: schedule.Schedule = 1.0, verbosity: int = 0):
    """The generalisation of decoupled AdamW and unfactored Adafactor (reference:
    axlearn/common/optimizers.py:1760-2090)::

        g_s   = ema(g, gradient_ema_decay)                   (optional, optionally debiased)
        g2_s  = ema(g^2 + eps_square, gradient_square_ema_decay)
        raw   = g_s / (sqrt(g2_s) + eps);  clipped to raw_update_clipping_threshold (block RMS)
        u     = ema(raw, update_ema_decay)                    (optional)
        u     = adam_update_transformation(u)                 (optional)
        delta = -update_schedule(t) * (learning_rate * u + weight_decay * scale_p * p)
    """
    sched = schedule.as_schedule_fn(update_schedule)
    inner = maybe_instantiate(adam_update_transformation) if adam_update_transformation is not None else None
    clip = clip_by_block_rms(raw_update_clipping_threshold)

    def zeros(params):
        return tree_map(lambda p: torch.zeros_like(p.value, dtype=torch.float32), params, is_leaf=_is_opt_param)

    def init(params):
        state = AdastarState(
            _count0(), None if gradient_ema_decay is None else zeros(params), zeros(params),
            None if update_ema_decay is None else zeros(params))
        return (state, inner.init(params)) if inner is not None else state

    def moment(x, acc, decay, debias, t):
        if decay is None:
            return x
        acc.mul_(decay).add_(x, alpha=1 - decay)
        return acc / (1 - decay ** t) if debias else acc.clone()

    def update(updates, state, params=None):
        if params is None:
            raise ValueError("adastar requires params")
        inner_state = None
        if inner is not None:
            state, inner_state = state
        count = _inc(state.count)
        t = int(count)
        g_ema = state.gradient_ema if state.gradient_ema is not None else tree_map(lambda _: None, state.gradient_square_ema)
        u_ema = state.update_ema if state.update_ema is not None else tree_map(lambda _: None, state.gradient_square_ema)

        def raw(g, m, v):
            g = g.float()
            gs = moment(g, m, gradient_ema_decay, gradient_ema_debias, t)
            g2 = moment(g * g + eps_square, v, gradient_square_ema_decay, gradient_square_ema_debias, t)
            return gs / (g2.sqrt() + eps)

        raw_updates = _map_updates(raw, updates, g_ema, state.gradient_square_ema)
        raw_updates, _ = clip.update(raw_updates, None, params)
        if verbosity > 0:
            _summary("raw_update_norm", global_norm(raw_updates))
        smoothed = _map_updates(lambda u, acc: moment(u, acc, update_ema_decay, update_ema_debias, t), raw_updates, u_ema)
        if inner is not None:
            smoothed, inner_state = inner.update(smoothed, inner_state, params)
        scales = _weight_decay_scales(params, weight_decay_per_param_scale)
        s = sched(t)
        _summary("schedule_scale", s)
        out = _map_updates(
            lambda u, p, ws: -s * (learning_rate * u + (weight_decay * ws) * p.value.float()), smoothed, params, scales)
        new_state = AdastarState(count, state.gradient_ema, state.gradient_square_ema, state.update_ema)
        return out, ((new_state, inner_state) if inner is not None else new_state)

    def partition(specs):
        st = AdastarState(_count_spec(), None if gradient_ema_decay is None else _copy_specs(specs, torch.float32),
                          _copy_specs(specs, torch.float32),
                          None if update_ema_decay is None else _copy_specs(specs, torch.float32))
        return (st, inner.partition(specs)) if inner is not None else st

    return PartitionedGradientTransformation(init, update, partition)


def scale_by_param_block_rms(threshold: float = 1e-3) -> PartitionedGradientTransformation:
    """Scales each update by ``max(rms(param), threshold)``."""

    def fn(updates, params):
        return _map_updates(
            lambda g, p: g * torch.clamp(p.value.float().pow(2).mean().sqrt(), min=threshold).to(g.dtype),
            updates, params)

    return _stateless(fn)


def scale_by_trust_ratio(min_norm: float = 0.0, trust_coefficient: float = 1.0, eps: float = 0.0):
    """LARS/LAMB trust ratio ``||p|| / ||u||`` per parameter."""

    def fn(updates, params):
        def upd(g, p):
            pn = torch.clamp(p.value.float().norm(), min=min_norm)
            un = g.float().norm()
            ratio = trust_coefficient * pn / (un + eps)
            ratio = torch.where((pn == 0) | (un == 0), torch.ones_like(ratio), ratio)
            return g * ratio.to(g.dtype)

        return _map_updates(upd, updates, params)

    return _stateless(fn)


class FactoredState(NamedTuple):
    count: Tensor
    v_row: Any
    v_col: Any
    v: Any


def scale_by_factored_rms(factored: bool = True, decay_rate: float = 0.8, step_offset: int = 0,
                          min_dim_size_to_factor: int = 128, epsilon: float = 1e-30):
    """Adafactor second-moment estimate, factored over the two largest dims of big tensors
    (reference: axlearn/common/factorized_rms.py:73)."""

    decay_fn = maybe_instantiate(decay_rate) if not isinstance(decay_rate, (int, float)) else None

    def factored_dims(shape):
        if not factored or len(shape) < 2:
            return None
        order = sorted(range(len(shape)), key=lambda i: shape[i])
        if shape[order[-2]] < min_dim_size_to_factor:
            return None
        return order[-2], order[-1]

    def init(params):
        def mk(p, which):
            fd = factored_dims(p.value.shape)
            shape = list(p.value.shape)
            if fd is None:
                return torch.zeros_like(p.value, dtype=torch.float32) if which == "v" else torch.zeros(1, device=p.value.device)
            if which == "v":
                return torch.zeros(1, device=p.value.device)
            drop = fd[0] if which == "row" else fd[1]
            shape.pop(drop)
            return torch.zeros(shape, dtype=torch.float32, device=p.value.device)

        m = lambda which: tree_map(lambda p: mk(p, which), params, is_leaf=_is_opt_param)
        return FactoredState(_count0(), m("row"), m("col"), m("v"))

    def update(updates, state, params=None):
        count = _inc(state.count)
        t = float(int(count) - step_offset)
        if callable(decay_fn):
            decay = float(decay_fn(int(count)))
        else:
            decay = 1.0 - t ** (-decay_rate) if t > 0 else 0.0

        def upd(g, vr, vc, v):
            gf = g.float()
            g2 = gf * gf + epsilon
            fd = factored_dims(g.shape)
            if fd is None:
                v.mul_(decay).add_(g2, alpha=1 - decay)
                return (gf * torch.rsqrt(v)).to(g.dtype)
            d0, d1 = fd
            vr.mul_(decay).add_(g2.mean(dim=d0), alpha=1 - decay)
            vc.mul_(decay).add_(g2.mean(dim=d1), alpha=1 - decay)
            # vr dropped d0 (keeps d1); vc dropped d1 (keeps d0).
            red = vc.mean(dim=(d0 if d0 < d1 else d0 - 1), keepdim=True)
            row_factor = torch.rsqrt(vc / red).unsqueeze(d1)
            col_factor = torch.rsqrt(vr).unsqueeze(d0)
            return (gf * row_factor * col_factor).to(g.dtype)

        out = _map_updates(upd, updates, state.v_row, state.v_col, state.v)
        return out, FactoredState(count, state.v_row, state.v_col, state.v)

    def partition(specs):
        any_spec = lambda s: OptStateSpec(shape=None, dtype=torch.float32, mesh_axes=None)
        m = tree_map(any_spec, specs, is_leaf=_is_spec)
        return FactoredState(_count_spec(), m, m, m)

    return PartitionedGradientTransformation(init, update, partition)


def clip_by_block_rms(threshold: Optional[float]) -> PartitionedGradientTransformation:
    """Scales each update tensor so that its RMS is at most ``threshold``."""

    def fn(updates, params):
        if threshold is None:
            return updates

        def upd(g):
            rms = g.float().pow(2).mean().sqrt()
            return g * torch.clamp(threshold / rms.clamp_min(1e-30), max=1.0).to(g.dtype)

        return _map_updates(upd, updates)

    return _stateless(fn)


def adafactor_optimizer(learning_rate: schedule.Schedule, *, b1: Optional[float] = None, b2: float = 0.8,
                        multiply_by_parameter_scale: bool = True, clipping_threshold: Optional[float] = 1.0,
                        dtype_momentum: Any = torch.float32, weight_decay: Optional[float] = None,
                        weight_decay_scale_by_learning_rate_exponent: Optional[float] = None,
                        weight_decay_per_param_scale: Optional[Callable] = None, eps: float = 1e-30,
                        factored: bool = True, apply_scale_by_trust_ratio: bool = False):
    links = [scale_by_factored_rms(factored=factored, decay_rate=b2, epsilon=eps)]
    if clipping_threshold is not None:
        links.append(clip_by_block_rms(clipping_threshold))
    if apply_scale_by_trust_ratio:
        links.append(scale_by_trust_ratio())
    links.append(scale_by_schedule(learning_rate))
    if multiply_by_parameter_scale:
        links.append(scale_by_param_block_rms())
    if b1:
        links.append(ema(decay=b1, debias=False, accumulator_dtype=dtype_momentum))
    if weight_decay:
        links.append(add_decayed_weights(
            weight_decay, learning_rate_exponent=weight_decay_scale_by_learning_rate_exponent,
            learning_rate=learning_rate, per_param_scale=weight_decay_per_param_scale))
    links.append(scale(-1.0))
    return chain(*links)


# ------------------------------------------------------------------------------------------
# EMA.
# ------------------------------------------------------------------------------------------


class EmaState(NamedTuple):
    count: Tensor
    ema: Any


def ema(decay: schedule.Schedule, debias: bool = True, accumulator_dtype: Optional[torch.dtype] = None):
    """Replaces updates by their exponential moving average."""
    decay_fn = schedule.as_schedule_fn(decay)

    def init(params):
        return EmaState(_count0(), tree_map(lambda p: torch.zeros_like(p.value, dtype=accumulator_dtype or p.value.dtype), params, is_leaf=_is_opt_param))

    def update(updates, state, params=None):
        count = _inc(state.count)
        d = decay_fn(int(count))

        def upd(g, e):
            e.mul_(d).add_(g.to(e.dtype), alpha=1 - d)
            out = e / (1 - d ** int(count)) if debias else e
            return out.to(g.dtype)

        return _map_updates(upd, updates, state.ema), EmaState(count, state.ema)

    return PartitionedGradientTransformation(init, update, lambda specs: EmaState(_count_spec(), _copy_specs(specs, accumulator_dtype)))


class ParamEmaState(NamedTuple):
    count: Tensor
    ema: Any


def param_ema(*, decay: Optional[schedule.Schedule] = None) -> PartitionedGradientTransformation:
    """Tracks an EMA of the *parameters* (updates pass through unchanged)."""
    if decay is None:
        return _stateless(lambda u, p: u)
    decay_fn = schedule.as_schedule_fn(decay)

    def init(params):
        return ParamEmaState(_count0(), tree_map(lambda p: p.value.detach().clone().float(), params, is_leaf=_is_opt_param))

    def update(updates, state, params):
        count = _inc(state.count)
        d = decay_fn(int(count))
        tree_map(lambda e, p: e.mul_(d).add_(p.value.detach().to(e.dtype), alpha=1 - d), state.ema, params,
                 is_leaf=lambda x: isinstance(x, (torch.Tensor, OptParam)))
        return updates, ParamEmaState(count, state.ema)

    return PartitionedGradientTransformation(init, update, lambda specs: ParamEmaState(_count_spec(), _copy_specs(specs, torch.float32)))


# ------------------------------------------------------------------------------------------
# Clipping.
# ------------------------------------------------------------------------------------------


def global_norm(tree: Any, *, specs: Optional[Any] = None) -> Tensor:
    """``sqrt(sum ||leaf||^2)`` over all ranks' shards.

    With a mesh in scope, each leaf's local sum of squares is weighted by the inverse of its
    replication factor (from ``specs``' mesh axes) and the total is all-reduced over the mesh,
    so replicated tensors are counted once.
    """
    from axlearn_b200.parallel.grad_sync import sharded_sum_of_squares

    return torch.sqrt(sharded_sum_of_squares(tree, specs=specs))


def clip_by_global_norm(max_norm: Optional[float] = None, *, drop_norm: Optional[float] = None,
                        eps: float = 1e-8) -> PartitionedGradientTransformation:
    """Scales all updates by ``min(1, max_norm / (||g|| + eps))``."""
    if drop_norm is not None:
        return skip_and_clip_by_global_norm(inner=_stateless(lambda u, p: u), max_norm=max_norm, drop_norm=drop_norm, eps=eps)

    def fn(updates, params):
        specs = _current_param_specs()
        g_norm = global_norm(updates, specs=specs)
        _summary("gradient_norm", g_norm)
        if max_norm is None:
            return updates
        g_scale = torch.clamp(max_norm / (g_norm + eps), max=1.0)
        _summary("gradient_scale", g_scale)
        return _map_updates(lambda g: g * g_scale.to(g.dtype), updates)

    tx = _stateless(fn)
    tx.clip_spec = (max_norm, eps) if max_norm is not None else None
    return tx


class SkipClipState(NamedTuple):
    nonvalid_count: Tensor
    inner_state: Any
    grad_norm_ema: Optional[Tensor] = None
    grad_norm_square_ema: Optional[Tensor] = None
    count: Optional[Tensor] = None
    drop_stats: Optional[dict] = None


def skip_and_clip_by_global_norm(inner: Any, *, drop_norm: Optional[Any] = None, max_norm: Optional[float] = None,
                                 grad_norm_ema_decay: Optional[float] = None, eps: float = 1e-8):
    """Skips the whole step (updates zeroed, inner state untouched) when the gradient norm is
    non-finite or exceeds ``drop_norm``; otherwise clips to ``max_norm`` and applies ``inner``.

    ``drop_norm`` may be a float or a callable ``(count, mean, stddev) -> {name: threshold}``
    evaluated on an EMA of past norms (adaptive thresholds).
    """
    inner = maybe_instantiate(inner)
    use_ema = grad_norm_ema_decay is not None

    def init(params):
        return SkipClipState(
            nonvalid_count=_count0(), inner_state=inner.init(params),
            grad_norm_ema=torch.zeros(()) if use_ema else None,
            grad_norm_square_ema=torch.zeros(()) if use_ema else None,
            count=_count0() if use_ema else None,
            drop_stats={} if use_ema else None,
        )

    def update(updates, state, params):
        specs = _current_param_specs()
        g_norm = global_norm(updates, specs=specs)
        gn = float(g_norm)
        _summary("gradient_norm", g_norm)
        is_finite = math.isfinite(gn)
        valid = is_finite
        new_ema, new_sq, new_count = state.grad_norm_ema, state.grad_norm_square_ema, state.count
        if drop_norm is not None:
            if callable(drop_norm) and use_ema:
                mean = float(state.grad_norm_ema)
                var = max(float(state.grad_norm_square_ema) - mean**2, 0.0)
                thresholds = drop_norm(count=int(state.count), mean=mean, stddev=math.sqrt(var))
                valid = valid and all(gn < float(t) for t in thresholds.values())
            else:
                valid = valid and gn < float(drop_norm)
        if use_ema and valid:
            d = grad_norm_ema_decay
            c = int(state.count) + 1
            new_ema = d * state.grad_norm_ema + (1 - d) * gn if int(state.count) > 0 else torch.tensor(gn)
            new_sq = d * state.grad_norm_square_ema + (1 - d) * gn * gn if int(state.count) > 0 else torch.tensor(gn * gn)
            new_count = torch.tensor(c, dtype=torch.int32)
        if not valid:
            _summary("is_valid_step", 0.0)
            zero = _map_updates(torch.zeros_like, updates)
            return zero, state._replace(nonvalid_count=_inc(state.nonvalid_count))
        _summary("is_valid_step", 1.0)
        if max_norm is not None:
            g_scale = min(1.0, max_norm / (gn + eps))
            _summary("gradient_scale", g_scale)
            updates = _map_updates(lambda g: g * g_scale, updates)
        out, inner_state = inner.update(updates, state.inner_state, params)
        return out, SkipClipState(state.nonvalid_count, inner_state, new_ema, new_sq, new_count, state.drop_stats)

    def partition(specs):
        s = OptStateSpec(shape=(), dtype=torch.float32, mesh_axes=PartitionSpec())
        return SkipClipState(_count_spec(), inner.partition(specs), s if use_ema else None,
                             s if use_ema else None, _count_spec() if use_ema else None, {} if use_ema else None)

    return PartitionedGradientTransformation(init, update, partition)


def drop_norm_by_grad_norm_ema(multipliers: Sequence[float] = (20, 40, 100)):
    """Adaptive thresholds ``mean * k`` for ``skip_and_clip_by_global_norm``."""

    def fn(count, mean, stddev):
        return {f"ema_x{k}": (mean * k if count > 0 else float("inf")) for k in multipliers}

    return fn


def drop_norm_by_grad_norm_stddev(min_count: int = 500, multipliers: Sequence[float] = (20, 40, 100)):
    def fn(count, mean, stddev):
        return {f"stddev_x{k}": (mean + stddev * k if count >= min_count else float("inf")) for k in multipliers}

    return fn


# ------------------------------------------------------------------------------------------
# Offload.
# ------------------------------------------------------------------------------------------


def offload_optimizer(optimizer: Any, *, pattern: Union[str, re.Pattern] = ".*",
                      offload_src: str = "device", offload_dst: str = "pinned_host"):
    """Keeps optimizer-state tensors whose path matches ``pattern`` in pinned host memory
    between steps; they are copied to the device for the update and back afterwards."""
    inner = maybe_instantiate(optimizer)
    pat = re.compile(pattern) if isinstance(pattern, str) else pattern
    del offload_src, offload_dst

    def to_host(state):
        paths = tree_paths(state)

        def mv(x, path):
            if isinstance(x, torch.Tensor) and x.is_cuda and x.dim() > 0 and pat.fullmatch(path):
                host = torch.empty(x.shape, dtype=x.dtype, device="cpu", pin_memory=True)
                host.copy_(x, non_blocking=True)
                host._axb_device = x.device  # pylint: disable=protected-access
                return host
            return x

        return tree_map(mv, state, paths)

    def to_device(state):
        def mv(x):
            dev = getattr(x, "_axb_device", None) if isinstance(x, torch.Tensor) else None
            return x.to(dev, non_blocking=True) if dev is not None else x

        return tree_map(mv, state)

    def init(params):
        return to_host(inner.init(params))

    def update(updates, state, params):
        out, new_state = inner.update(updates, to_device(state), params)
        return out, to_host(new_state)

    return PartitionedGradientTransformation(init, update, inner.partition)


# ------------------------------------------------------------------------------------------
# Param-spec context (lets norm computations know how each leaf is sharded).
# ------------------------------------------------------------------------------------------

_param_specs_stack: list = []


class param_specs_scope:  # pylint: disable=invalid-name
    """Declares the ParameterSpec tree matching the updates being transformed."""

    def __init__(self, specs: Any):
        self._specs = specs

    def __enter__(self):
        _param_specs_stack.append(self._specs)

    def __exit__(self, *exc):
        _param_specs_stack.pop()


def _current_param_specs() -> Optional[Any]:
    return _param_specs_stack[-1] if _param_specs_stack else None


def apply_updates(params: Any, updates: Any) -> Any:
    """``p + u`` per leaf (params are plain tensors); ``None`` updates leave p unchanged."""
    return tree_map(
        lambda p, u: p if u is None else p + u.to(p.dtype), params, updates,
        is_leaf=lambda x: x is None or isinstance(x, torch.Tensor))
