"""MoE feed-forward layer on the GPU kernels (bf16) against the fp32 reference path."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_moe_layer_bf16_matches_fp32_reference():
    from axlearn_b200.common import prng
    from axlearn_b200.common.mixture_of_experts import Top2Gating, TransformerFeedForwardMoE
    from axlearn_b200.common.module import functional
    from axlearn_b200.common.utils import tree_map
    from axlearn_b200.ops import cuda_ops, dispatch

    cfg = TransformerFeedForwardMoE.default_config().set(
        name="moe", input_dim=256, hidden_dim=512, num_experts=4, num_groups=2, activation=("nn.silu", "linear"),
        structure="nonorm", gating=Top2Gating.default_config().set(train_capacity_factor=2.0))
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0))
    # Both paths see the same bf16-rounded values, so the router takes identical decisions.
    params = tree_map(lambda t: t.cuda().bfloat16().float(), params)
    x = torch.randn(4, 64, 256, device="cuda").bfloat16().float()

    def run(p, inp):
        p = tree_map(lambda t: t.detach().clone().requires_grad_(True), p)
        out, oc = functional(layer, prng.PRNGKey(1), p, [inp], is_training=True, drop_output_collections=())
        (out.float().square().mean() + oc.module_outputs["aux_loss"]).backward()
        return out, p

    with dispatch.use_reference_ops():
        ref_out, ref_p = run(params, x)
    # bf16 activations and weights; the router (gate_weight) stays fp32 inside the layer.
    before = cuda_ops.launch_count
    bf_params = tree_map(lambda t: t.bfloat16(), params)
    out, p = run(bf_params, x.bfloat16())
    torch.cuda.synchronize()
    cuda_ops.check_status()
    assert cuda_ops.launch_count > before, "the expert GEMMs must run on the CUDA kernels"
    scale = ref_out.abs().max().item()
    assert (out.float() - ref_out).abs().max().item() < 3e-2 * scale
    for name in ("wi_0_weight", "wo_weight"):
        g, r = p[name].grad.float(), ref_p[name].grad
        assert (g - r).abs().max().item() < 6e-2 * r.abs().max().item(), name


def test_dispatch_combine_kernels_match_torch_formulation():
    from axlearn_b200.ops import cuda_ops, dispatch, moe_ops

    torch.manual_seed(0)
    t, k, m, rows = 300, 2, 256, 1024
    # Unique destinations with some dropped assignments.
    perm = torch.randperm(rows, device="cuda")[:t * k].reshape(t, k).to(torch.int32)
    drop = torch.rand(t, k, device="cuda") < 0.2
    dest = torch.where(drop, torch.full_like(perm, -1), perm)
    x = torch.randn(t, m, device="cuda").bfloat16().requires_grad_(True)
    y = torch.randn(rows, m, device="cuda").bfloat16().requires_grad_(True)
    w = torch.rand(t, k, device="cuda").requires_grad_(True)
    gd = torch.randn(rows, m, device="cuda").bfloat16()
    gc = torch.randn(t, m, device="cuda").bfloat16()

    def run():
        d = moe_ops.dispatch(x, dest, rows)
        c = moe_ops.combine(y, w, dest)
        grads = torch.autograd.grad([d, c], [x, y, w], [gd, gc])
        return d, c, grads

    d, c, g = run()
    with dispatch.use_reference_ops():
        d_ref, c_ref, g_ref = run()
    torch.cuda.synchronize()
    cuda_ops.check_status()
    assert torch.equal(d, d_ref)
    assert (c.float() - c_ref.float()).abs().max() < 3e-2
    for a, b in zip(g, g_ref):
        assert (a.float() - b.float()).abs().max() < 5e-2 * max(1.0, b.float().abs().max().item())


def test_peer_exchange_on_one_gpu_matches_local_dispatch(monkeypatch):
    """The push / pull kernels and their hand-shake with a group of one (this GPU is its own
    peer) must reproduce the local gather / combine path, forward and backward."""
    from axlearn_b200.common import prng
    from axlearn_b200.common.mixture_of_experts import Top2Gating, TransformerFeedForwardMoE
    from axlearn_b200.common.module import functional
    from axlearn_b200.common.utils import tree_map
    from axlearn_b200.ops import cuda_ops

    cfg = TransformerFeedForwardMoE.default_config().set(
        name="moe", input_dim=256, hidden_dim=512, num_experts=4, num_groups=2, activation=("nn.silu", "linear"),
        structure="nonorm", gating=Top2Gating.default_config().set(train_capacity_factor=1.0))
    layer = cfg.instantiate(parent=None)
    params = tree_map(lambda t: t.cuda().bfloat16(), layer.initialize_parameters_recursively(prng.PRNGKey(0)))
    x = torch.randn(4, 64, 256, device="cuda").bfloat16()

    def run():
        p = tree_map(lambda t: t.detach().clone().requires_grad_(True), params)
        xin = x.clone().requires_grad_(True)
        outs = []
        for _ in range(2):   # twice: the second round exercises the "box is free again" waits
            out, oc = functional(layer, prng.PRNGKey(1), p, [xin], is_training=True, drop_output_collections=())
            (out.float().square().mean() + oc.module_outputs["aux_loss"]).backward()
            outs.append(out.detach().float())
        return outs, p, xin.grad.float()

    monkeypatch.setenv("AXB_MOE_PEER_EXCHANGE", "0")
    ref_outs, ref_p, ref_dx = run()
    monkeypatch.setenv("AXB_MOE_PEER_EXCHANGE", "force")
    before = cuda_ops.launch_count
    outs, p, dx = run()
    torch.cuda.synchronize()
    cuda_ops.check_status()
    assert cuda_ops.launch_count - before > 20
    for a, b in zip(outs, ref_outs):
        assert torch.equal(a, b)
    assert torch.equal(dx, ref_dx)
    for name in ("wi_0_weight", "wo_weight", "gate_weight"):
        assert torch.equal(p[name].grad, ref_p[name].grad), name
