"""Optimizer algebra against closed forms and torch.optim, schedules, update transformations."""

import math

import pytest
import torch

from axlearn_b200.common import optimizers as opt
from axlearn_b200.common import schedule
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.optimizer_base import OptParam
from axlearn_b200.common.update_transformation import (
    ConditionalUpdateTransformation,
    OverrideInplaceUpdateTransformation,
    conditional_update,
    override_inplace_update,
)


def _params(seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"a": {"weight": torch.randn(4, 3, generator=g)}, "b": {"bias": torch.randn(3, generator=g)}}


def _opt_params(params):
    return {k: {kk: OptParam(vv, None, None) for kk, vv in v.items()} for k, v in params.items()}


def _run(tx, params, grads_per_step):
    params = {k: {kk: vv.clone() for kk, vv in v.items()} for k, v in params.items()}
    state = tx.init(_opt_params(params))
    for grads in grads_per_step:
        updates, state = tx.update(grads, state, _opt_params(params))
        for k in params:
            for kk in params[k]:
                if updates[k][kk] is not None:
                    params[k][kk] = params[k][kk] + updates[k][kk]
    return params, state


def _grads(n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [{"a": {"weight": torch.randn(4, 3, generator=g)}, "b": {"bias": torch.randn(3, generator=g)}}
            for _ in range(n)]


def test_adamw_matches_torch():
    params, grads = _params(), _grads(5)
    tx = opt.adamw_optimizer(1e-2, b1=0.9, b2=0.99, eps=1e-8, weight_decay=0.1)
    got, _ = _run(tx, params, grads)
    ref = [torch.nn.Parameter(params["a"]["weight"].clone()), torch.nn.Parameter(params["b"]["bias"].clone())]
    o = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    for g in grads:
        ref[0].grad, ref[1].grad = g["a"]["weight"].clone(), g["b"]["bias"].clone()
        o.step()
    torch.testing.assert_close(got["a"]["weight"], ref[0].data, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(got["b"]["bias"], ref[1].data, rtol=1e-5, atol=1e-6)


def test_adamw_decoupled_closed_form_and_state_layout():
    params, grads = _params(), _grads(3)
    sched = schedule.cosine_with_linear_warmup(peak_lr=1.0, warmup_steps=2, max_step=10, alpha=0.1)
    tx = opt.adamw_decoupled_optimizer(3e-3, b1=0.9, b2=0.95, eps=1e-8, update_schedule=sched, weight_decay=0.1)
    got, state = _run(tx, params, grads)
    p = params["a"]["weight"].clone()
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    for t, g in enumerate(grads, start=1):
        g = g["a"]["weight"]
        m = 0.9 * m + 0.1 * g
        v = 0.95 * v + 0.05 * g * g
        mh, vh = m / (1 - 0.9 ** t), v / (1 - 0.95 ** t)
        p = p - sched(t) * (3e-3 * mh / (vh.sqrt() + 1e-8) + 0.1 * p)
    torch.testing.assert_close(got["a"]["weight"], p, rtol=1e-5, atol=1e-6)
    # Chain state: scale_by_adam, lr schedule, decayed weights (stateless count), update schedule, scale.
    assert int(state[0].count) == 3 and int(state[1].count) == 3 and int(state[3].count) == 3
    assert state[0].mu["a"]["weight"].shape == (4, 3)


def test_adastar_reproduces_adamw_decoupled():
    params, grads = _params(), _grads(4)
    sched = schedule.cosine_with_linear_warmup(peak_lr=1.0, warmup_steps=2, max_step=10)
    ref, _ = _run(opt.adamw_decoupled_optimizer(3e-3, b1=0.9, b2=0.95, eps=1e-8, update_schedule=sched,
                                                weight_decay=0.05), params, grads)
    got, state = _run(opt.adastar_optimizer(
        3e-3, gradient_ema_decay=0.9, gradient_ema_debias=True, gradient_square_ema_decay=0.95,
        gradient_square_ema_debias=True, eps=1e-8, eps_square=0.0, raw_update_clipping_threshold=None,
        update_ema_decay=None, update_ema_debias=False, weight_decay=0.05, update_schedule=sched), params, grads)
    torch.testing.assert_close(got["a"]["weight"], ref["a"]["weight"], rtol=1e-5, atol=1e-6)
    assert state.update_ema is None and int(state.count) == 4


def test_adastar_update_ema_and_clipping():
    params, grads = _params(), _grads(3)
    got, state = _run(opt.adastar_optimizer(
        1e-2, gradient_ema_decay=None, gradient_ema_debias=False, gradient_square_ema_decay=0.8,
        gradient_square_ema_debias=True, eps=0.0, eps_square=1e-30, raw_update_clipping_threshold=1.0,
        update_ema_decay=0.9, update_ema_debias=False, update_schedule=1.0), params, grads)
    assert state.gradient_ema is None and state.update_ema["a"]["weight"].abs().sum() > 0
    assert not torch.equal(got["a"]["weight"], params["a"]["weight"])


def test_lion_and_sgd_momentum():
    params, grads = _params(), _grads(2)
    got, _ = _run(opt.lion_optimizer(1e-2, b1=0.9, b2=0.99), params, grads)
    m = torch.zeros(4, 3)
    p = params["a"]["weight"].clone()
    for g in grads:
        g = g["a"]["weight"]
        p = p - 1e-2 * torch.sign(0.9 * m + 0.1 * g)
        m = 0.99 * m + 0.01 * g
    torch.testing.assert_close(got["a"]["weight"], p)
    got, _ = _run(opt.sgd_optimizer(0.1, decouple_weight_decay=False, momentum=0.9), params, grads)
    ref = torch.nn.Parameter(params["a"]["weight"].clone())
    o = torch.optim.SGD([ref], lr=0.1, momentum=0.9)
    for g in grads:
        ref.grad = g["a"]["weight"].clone()
        o.step()
    torch.testing.assert_close(got["a"]["weight"], ref.data, rtol=1e-5, atol=1e-6)


def test_clip_by_global_norm_and_adafactor_runs():
    grads = _grads(1)[0]
    total = math.sqrt(sum(float(v.pow(2).sum()) for d in grads.values() for v in d.values()))
    tx = opt.clip_by_global_norm(max_norm=0.5)
    out, _ = tx.update(grads, tx.init(_opt_params(_params())), _opt_params(_params()))
    new_total = math.sqrt(sum(float(v.pow(2).sum()) for d in out.values() for v in d.values()))
    assert total > 0.5 and abs(new_total - 0.5) < 1e-4
    got, _ = _run(opt.adafactor_optimizer(1e-2, b1=0.9, b2=0.8, multiply_by_parameter_scale=False,
                                          clipping_threshold=1.0), _params(), _grads(2))
    assert torch.isfinite(got["a"]["weight"]).all()


def test_skip_and_clip_skips_large_gradients():
    params = _params()
    big = {"a": {"weight": torch.full((4, 3), 100.0)}, "b": {"bias": torch.full((3,), 100.0)}}
    tx = opt.skip_and_clip_by_global_norm(opt.sgd_optimizer(0.1, decouple_weight_decay=False), drop_norm=10.0,
                                          max_norm=1.0)
    got, state = _run(tx, params, [big])
    assert torch.equal(got["a"]["weight"], params["a"]["weight"])
    got, _ = _run(tx, params, _grads(1))
    assert not torch.equal(got["a"]["weight"], params["a"]["weight"])


def test_schedules_are_one_based():
    s = schedule.cosine_with_linear_warmup(peak_lr=2.0, warmup_steps=4, max_step=12, alpha=0.1)
    assert abs(s(1) - 0.5) < 1e-6 and abs(s(4) - 2.0) < 1e-6 and abs(s(12) - 0.2) < 1e-6
    w = schedule.warmup_stable_decay(peak_lr=1.0, max_step=20, warmup_steps=5)
    assert w(5) == pytest.approx(1.0) and w(10) == pytest.approx(1.0) and w(20) < 1.0
    st = schedule.stepwise(sub=[0.1, 0.01], start_step=[10])
    assert st(9) == pytest.approx(0.1) and st(10) == pytest.approx(0.01)


def test_conditional_update_runs_every_k_steps():
    params, grads = _params(), _grads(4)
    tx = conditional_update(opt.sgd_optimizer(0.1, decouple_weight_decay=False), update_every_k=2)
    p1, _ = _run(tx, params, grads[:1])
    assert torch.equal(p1["a"]["weight"], params["a"]["weight"])            # step 1: no-op
    p2, state = _run(tx, params, grads[:2])
    torch.testing.assert_close(p2["a"]["weight"], params["a"]["weight"] - 0.1 * grads[1]["a"]["weight"])
    assert int(state.count) == 2
    cfg = ConditionalUpdateTransformation.default_config().set(
        inner=config_for_function(opt.sgd_optimizer).set(learning_rate=0.1, decouple_weight_decay=False),
        update_every_k=2)
    p2b, _ = _run(cfg.instantiate(), params, grads[:2])
    torch.testing.assert_close(p2b["a"]["weight"], p2["a"]["weight"])


def test_override_inplace_takes_the_gradient_as_the_new_value():
    params, grads = _params(), _grads(1)
    tx = override_inplace_update(opt.sgd_optimizer(0.1, decouple_weight_decay=False), rules=["b/bias"])
    got, _ = _run(tx, params, grads)
    torch.testing.assert_close(got["b"]["bias"], grads[0]["b"]["bias"])
    torch.testing.assert_close(got["a"]["weight"], params["a"]["weight"] - 0.1 * grads[0]["a"]["weight"])
    cfg = OverrideInplaceUpdateTransformation.default_config().set(
        transformation=config_for_function(opt.sgd_optimizer).set(learning_rate=0.1, decouple_weight_decay=False),
        rules=[".*bias"])
    got2, _ = _run(cfg.instantiate(), params, grads)
    torch.testing.assert_close(got2["b"]["bias"], grads[0]["b"]["bias"])
