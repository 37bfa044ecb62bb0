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


@pytest.mark.parametrize("g,s,e,k,cap,logit_cap,sigmoid", [
    (2, 300, 8, 2, 60, 0.0, False),       # Mixtral-like: 8 experts, top-2, some tokens dropped
    (1, 4096, 8, 2, 2048, 0.0, False),
    (3, 1111, 16, 1, 50, 5.0, False),     # top-1 with a logit cap
    (2, 700, 128, 8, 64, 0.0, False),     # Qwen3-like: 128 experts, top-8
    (1, 513, 40, 4, 1000, 0.0, True),     # sigmoid scores, nothing dropped
    (1, 37, 5, 3, 7, 0.0, False),         # tiny, fewer tokens than one chunk
])
def test_routing_kernel_matches_torch_statements(g, s, e, k, cap, logit_cap, sigmoid):
    """Scores, top-k, capacity positions (choice-major priority), counts, score sums and the
    log-sum-exp from one kernel, and the gradient of the logits from its backward kernel."""
    from axlearn_b200.ops import moe_ops

    torch.manual_seed(0)
    logits = (torch.randn(g, s, e, device="cuda") * 2).requires_grad_()
    index, gate, slot, counts, sums, lse = moe_ops.topk_gate(logits, k, cap, logit_cap=logit_cap, sigmoid=sigmoid)
    ref_logits = logits.detach().clone().requires_grad_()
    r_index, r_gate, r_slot, r_counts, r_sums, r_lse = moe_ops.topk_gate_reference(ref_logits, k, cap, logit_cap, sigmoid)
    # Ties between equal scores are vanishingly rare with random floats: indices must agree.
    assert torch.equal(index, r_index)
    assert torch.equal(slot, r_slot)
    assert torch.equal(counts, r_counts)
    # (the kernel's tanh of the logit cap is the fast approximation)
    tol = 2e-3 if logit_cap > 0 else 1e-6
    assert torch.allclose(gate, r_gate, atol=tol, rtol=1e-5)
    assert torch.allclose(sums, r_sums, atol=1e-3 + s * tol, rtol=1e-5)
    assert torch.allclose(lse, r_lse, atol=max(tol, 1e-5), rtol=1e-5)
    # Every expert's kept positions are exactly 0 .. min(count, capacity) - 1.
    for gi in range(g):
        for ei in range(min(e, 4)):
            pos = slot[gi][index[gi] == ei]
            kept = pos[pos >= 0].sort().values
            assert torch.equal(kept, torch.arange(kept.numel(), device="cuda"))
            assert kept.numel() == min(int(counts[gi, :, ei].sum()), cap)
    w_gate = torch.randn_like(gate)
    w_sums = torch.randn_like(sums)
    w_lse = torch.randn_like(lse)
    ((gate * w_gate).sum() + (sums * w_sums).sum() + (lse * w_lse).sum()).backward()
    ((r_gate * w_gate).sum() + (r_sums * w_sums).sum() + (r_lse * w_lse).sum()).backward()
    assert torch.allclose(logits.grad, ref_logits.grad, atol=2e-5 if logit_cap == 0 else 5e-3, rtol=1e-4)


def test_gating_layers_use_the_routing_kernel_and_match_the_step_by_step_path():
    from axlearn_b200.common import prng
    from axlearn_b200.common.mixture_of_experts import Top2Gating, TopKGating
    from axlearn_b200.common.module import functional
    from axlearn_b200.ops import dispatch

    torch.manual_seed(1)
    for cfg in (Top2Gating.default_config().set(name="g", num_experts=8, train_capacity_factor=1.0),
                TopKGating.default_config().set(name="g", num_experts=16, num_experts_per_token=4,
                                                train_capacity_factor=2.0)):
        layer = cfg.instantiate(parent=None)
        logits = torch.randn(1, 2, 512, cfg.num_experts, device="cuda")
        a = logits.clone().requires_grad_()
        out_a, _ = functional(layer, prng.PRNGKey(0), {}, [a], is_training=True)
        b = logits.clone().requires_grad_()
        with dispatch.use_reference_ops():
            out_b, _ = functional(layer, prng.PRNGKey(0), {}, [b], is_training=True)
        assert torch.equal(out_a.expert_index, out_b.expert_index) and torch.equal(out_a.slot, out_b.slot)
        assert torch.allclose(out_a.weight, out_b.weight, atol=1e-5)
        assert torch.allclose(out_a.load_balance_loss, out_b.load_balance_loss, rtol=1e-4)
        assert torch.allclose(out_a.router_z_loss, out_b.router_z_loss, rtol=1e-4)
        wa = torch.randn_like(out_a.weight)
        ((out_a.weight * wa).sum() + out_a.load_balance_loss + out_a.router_z_loss).backward()
        ((out_b.weight * wa).sum() + out_b.load_balance_loss + out_b.router_z_loss).backward()
        assert torch.allclose(a.grad, b.grad, atol=2e-5, rtol=1e-3)
