"""MoE routing and the MoE feed-forward layer against a dense one-hot/einsum formulation."""

import math

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.mixture_of_experts import (
    Top2Gating,
    TopKGating,
    TransformerFeedForwardMoE,
    _compute_expert_capacity,
)
from axlearn_b200.common.module import functional


def _dense_top2(logits, capacity):
    """The GShard formulation with one-hot masks and cumulative sums (what the reference
    computes, axlearn/common/mixture_of_experts.py:526-640), written independently here."""
    o, g, s, e = logits.shape
    gates = torch.softmax(logits.float(), -1)
    i1 = gates.argmax(-1)
    m1 = torch.nn.functional.one_hot(i1, e).float()
    g_wo1 = gates * (1 - m1)
    i2 = g_wo1.argmax(-1)
    m2 = torch.nn.functional.one_hot(i2, e).float()
    g1 = (gates * m1).sum(-1)
    g2 = (g_wo1 * m2).sum(-1)
    den = g1 + g2 + 1e-9
    g1, g2 = g1 / den, g2 / den
    aux = (m1.mean(-2) * gates.mean(-2)).mean() * e * e
    p1 = m1.cumsum(-2) - m1
    m1 = m1 * (p1 < capacity)
    p1 = (p1 * m1).sum(-1)
    c1 = m1.sum(-2, keepdim=True)
    p2 = m2.cumsum(-2) - m2 + c1
    m2 = m2 * (p2 < capacity)
    p2 = (p2 * m2).sum(-1)
    g1 = g1 * m1.sum(-1)
    g2 = g2 * m2.sum(-1)
    comb = (g1[..., None, None] * m1[..., None] * torch.nn.functional.one_hot(p1.long(), capacity)[..., None, :]
            + g2[..., None, None] * m2[..., None] * torch.nn.functional.one_hot(p2.long(), capacity)[..., None, :])
    return comb, aux


def _run(layer_cfg, method_inputs, *, is_training=True, params=None, method="forward"):
    layer = layer_cfg.set(name="test").instantiate(parent=None)
    if params is None:
        params = layer.initialize_parameters_recursively(prng.PRNGKey(0))
    out, oc = functional(layer, prng.PRNGKey(1), params, method_inputs, is_training=is_training, method=method,
                         drop_output_collections=())
    return layer, params, out, oc


def test_expert_capacity():
    assert _compute_expert_capacity(group_size=64, num_experts=8, expert_capacity=None, capacity_factor=2.0) == 16
    assert _compute_expert_capacity(group_size=64, num_experts=8, expert_capacity=20, capacity_factor=2.0) == 20
    assert _compute_expert_capacity(group_size=64, num_experts=8, expert_capacity=3, capacity_factor=None) == 3
    with pytest.raises(ValueError):
        _compute_expert_capacity(group_size=64, num_experts=8, expert_capacity=None, capacity_factor=None)


@pytest.mark.parametrize("capacity_factor", [2.0, 0.5])
def test_top2_gating_matches_dense_formulation(capacity_factor):
    torch.manual_seed(0)
    o, g, s, e = 2, 3, 16, 4
    logits = torch.randn(o, g, s, e) * 2
    cfg = Top2Gating.default_config().set(num_experts=e, train_capacity_factor=capacity_factor)
    _, _, routing, oc = _run(cfg, [logits])
    cap = int(s * capacity_factor / e)
    assert routing.expert_capacity == cap
    comb, aux = _dense_top2(logits, cap)
    assert torch.allclose(routing.combine_tensor(), comb, atol=1e-6)
    assert torch.equal(routing.dispatch_tensor(), comb > 0)
    assert torch.allclose(routing.load_balance_loss, aux, atol=1e-6)
    if capacity_factor < 1:
        assert (routing.slot < 0).any()          # tokens were dropped
    counts = (routing.slot >= 0).sum(-1)
    for i in range(3):
        assert oc.summaries[f"dispatch_{i}"] == (counts == i).sum()


def test_topk_gating_priority_order_and_weights():
    torch.manual_seed(1)
    o, g, s, e, k = 1, 2, 12, 6, 3
    logits = torch.randn(o, g, s, e)
    cfg = TopKGating.default_config().set(num_experts=e, num_experts_per_token=k, train_capacity_factor=1.5)
    _, _, r, _ = _run(cfg, [logits])
    gates = torch.softmax(logits, -1)
    top = gates.topk(k, -1)
    assert torch.equal(r.expert_index, top.indices)
    cap = int(s * 1.5 / e)
    # Brute force: fill experts choice by choice, token by token.
    for gi in range(g):
        fill = [0] * e
        for kk in range(k):
            for t in range(s):
                ex = int(top.indices[0, gi, t, kk])
                expect = fill[ex] if fill[ex] < cap else -1
                fill[ex] += 1
                assert int(r.slot[0, gi, t, kk]) == expect
    w = top.values / top.values.sum(-1, keepdim=True) * (r.slot >= 0)
    assert torch.allclose(r.weight, w, atol=1e-6)
    assigned = torch.nn.functional.one_hot(top.indices, e).amax(-2).float()
    aux = (assigned.mean(-2) * gates.mean(-2)).mean() * e * e / k
    assert torch.allclose(r.load_balance_loss, aux, atol=1e-6)


def test_dispatch_combine_roundtrip_equals_einsum():
    torch.manual_seed(2)
    o, g, s, e, m = 2, 2, 8, 4, 5
    logits = torch.randn(o, g, s, e)
    cfg = Top2Gating.default_config().set(num_experts=e, train_capacity_factor=1.0)
    layer, params, r, _ = _run(cfg, [logits])
    x = torch.randn(o, g, s, m)
    d = layer.dispatch(x, r)
    ref = torch.einsum("ogsec,ogsm->oegcm", r.dispatch_tensor().float(), x)
    assert torch.allclose(d, ref, atol=1e-6)
    y = torch.randn(o, e, g, r.expert_capacity, m)
    c = layer.combine(y, r)
    ref_c = torch.einsum("ogsec,oegcm->ogsm", r.combine_tensor(), y)
    assert torch.allclose(c, ref_c, atol=1e-5)


def _moe_cfg(**kw):
    kw.setdefault("gating", Top2Gating.default_config().set(train_capacity_factor=2.0))
    return TransformerFeedForwardMoE.default_config().set(
        input_dim=16, hidden_dim=32, num_experts=4, num_groups=2, activation=("nn.silu", "linear"), **kw)


def test_moe_layer_forward_matches_dense_reference_and_backprops():
    torch.manual_seed(3)
    cfg = _moe_cfg(structure="prenorm")
    x = torch.randn(4, 8, 16)
    layer, params, out, oc = _run(cfg, [x])
    # Dense reference with the same parameters.
    from axlearn_b200.ops import reference

    normed = torch.nn.functional.layer_norm(x, (16,), params["norm"]["scale"], params["norm"]["bias"], eps=1e-8) \
        if "bias" in params["norm"] else None
    layer_norm_out, _ = functional(layer.norm, None, params["norm"], [x], is_training=True)
    xs = layer_norm_out.reshape(1, 2, 16, 16)
    logits = torch.einsum("ogsm,me->ogse", xs, params["gate_weight"])
    comb, aux = _dense_top2(logits, int(16 * 2.0 / 4))
    disp = (comb > 0).float()
    ein = torch.einsum("ogsec,ogsm->oegcm", disp, xs)
    h = torch.nn.functional.silu(torch.einsum("oegcm,emh->oegch", ein, params["wi_0_weight"])) * torch.einsum(
        "oegcm,emh->oegch", ein, params["wi_1_weight"])
    y = torch.einsum("oegch,ehm->oegcm", h, params["wo_weight"])
    ref = torch.einsum("ogsec,oegcm->ogsm", comb, y).reshape(4, 8, 16) + x
    assert torch.allclose(out, ref, atol=1e-5), (out - ref).abs().max()
    got_aux = oc.module_outputs["aux_loss"]
    assert torch.allclose(got_aux, aux * 0.01, atol=1e-7)
    del normed, reference

    # Gradients flow to the router and every expert that received tokens.
    params_g = {k: (v.clone().requires_grad_(True) if isinstance(v, torch.Tensor) else v) for k, v in params.items()
                if not isinstance(v, dict)}
    params_g.update({k: v for k, v in params.items() if isinstance(v, dict)})
    out2, oc2 = functional(layer, prng.PRNGKey(1), params_g, [x], is_training=True, drop_output_collections=())
    (out2.square().mean() + oc2.module_outputs["aux_loss"]).backward()
    assert params_g["gate_weight"].grad.abs().sum() > 0
    assert (params_g["wo_weight"].grad.abs().sum(dim=(1, 2)) > 0).all()


@pytest.mark.parametrize("structure", ["postnorm", "hybridnorm", "nonorm"])
def test_moe_layer_structures_run(structure):
    cfg = _moe_cfg(structure=structure, gating=TopKGating.default_config().set(num_experts_per_token=2))
    x = torch.randn(2, 8, 16)
    _, _, out, _ = _run(cfg, [x])
    assert out.shape == x.shape and torch.isfinite(out).all()


def test_routing_reference_function_matches_the_layer_statements():
    """``moe_ops.topk_gate_reference`` (the oracle of the routing kernel) agrees with the slot /
    count helpers the gating layers use."""
    import torch

    from axlearn_b200.common import mixture_of_experts as moe
    from axlearn_b200.ops import moe_ops

    torch.manual_seed(0)
    g, s, e, k, cap = 3, 200, 8, 2, 30
    logits = torch.randn(g, s, e)
    index, gate, slot, counts, sums, lse = moe_ops.topk_gate_reference(logits, k, cap)
    probs = torch.softmax(logits, -1)
    assert torch.equal(index, probs.topk(k, -1).indices)
    assert torch.allclose(gate, torch.gather(probs, -1, index))
    want_slot = moe._slots_in_priority_order(index.reshape(1, g, s, k), e, cap)  # pylint: disable=protected-access
    assert torch.equal(slot, want_slot.reshape(g, s, k))
    for j in range(k):
        assert torch.equal(counts[:, j], moe._expert_counts(index[..., j].reshape(1, g, s), e).reshape(g, e))  # pylint: disable=protected-access
    assert torch.allclose(sums, probs.sum(1)) and torch.allclose(lse, torch.logsumexp(logits, -1))
