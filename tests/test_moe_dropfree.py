"""Drop-free mixture of experts: routing, the padded sorted layout, grouped linear, and the layer
against a dense per-token loop."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.mixture_of_experts import (
    TopKBiasGating,
    TopKDropFreeGating,
    TransformerFeedForwardDropFreeMoE,
    convert_dense_to_moe_parameters,
)
from axlearn_b200.common.module import functional
from axlearn_b200.ops import moe_ops


def _layer(num_experts=4, k=2, dim=16, hidden=32, gating=None):
    cfg = TransformerFeedForwardDropFreeMoE.default_config().set(
        name="moe", input_dim=dim, hidden_dim=hidden, num_experts=num_experts,
        activation=("nn.silu", "linear"), structure="prenorm")
    cfg.gating = (gating or TopKDropFreeGating.default_config()).set(num_experts_per_token=k)
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    return layer, params


def _dense_oracle(layer, params, x):
    """Every token through its chosen experts, one at a time."""
    cfg = layer.config
    normed = torch.nn.functional.layer_norm(x, (cfg.input_dim,), params["norm"]["scale"], params["norm"]["bias"], eps=1e-8)
    logits = normed.reshape(-1, cfg.input_dim) @ params["gate_weight"]
    gates = torch.softmax(logits, dim=-1)
    w, idx = gates.topk(cfg.gating.num_experts_per_token, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    flat = normed.reshape(-1, cfg.input_dim)
    out = torch.zeros_like(flat)
    for t in range(flat.shape[0]):
        for j in range(idx.shape[1]):
            e = idx[t, j]
            h = torch.nn.functional.silu(flat[t] @ params["wi_0_weight"][e]) * (flat[t] @ params["wi_1_weight"][e])
            out[t] += w[t, j] * (h @ params["wo_weight"][e])
    return out.reshape(x.shape) + x


def test_padded_layout_properties():
    torch.manual_seed(0)
    experts = torch.randint(0, 6, (3, 50))
    experts[experts == 4] = 1                      # an empty expert
    dest, offsets, block_expert, rows = moe_ops.padded_group_layout(experts, 6)
    blk = moe_ops.GROUP_BLOCK
    assert rows % blk == 0 and offsets[-1] <= rows
    assert (offsets % blk == 0).all() and offsets[4] == offsets[5]
    flat, d = experts.reshape(-1), dest.long()
    assert d.unique().numel() == flat.numel()
    assert ((d >= offsets[flat.long()]) & (d < offsets[flat.long() + 1])).all()
    # Pair order is kept inside an expert's run.
    for e in range(6):
        mine = d[flat == e]
        assert (mine[1:] > mine[:-1]).all()
    for b, e in enumerate(block_expert.tolist()):
        if e >= 0:
            assert offsets[e] <= b * blk < offsets[e + 1]
        else:
            assert b * blk >= offsets[-1]


def test_dropfree_layer_matches_per_token_loop():
    layer, params = _layer()
    torch.manual_seed(1)
    x = torch.randn(2, 12, 16)
    out, oc = functional(layer, prng.PRNGKey(1), params, dict(inputs=x), is_training=True, drop_output_collections=())
    torch.testing.assert_close(out, _dense_oracle(layer, params, x), rtol=1e-4, atol=1e-5)
    assert "aux_loss" in oc.module_outputs


def test_dropfree_layer_gradients_flow_to_all_parts():
    layer, params = _layer()
    params = {k: (v.requires_grad_() if torch.is_tensor(v) else {kk: vv.requires_grad_() for kk, vv in v.items()})
              for k, v in params.items()}
    x = torch.randn(2, 8, 16, requires_grad=True)
    out, oc = functional(layer, prng.PRNGKey(1), params, dict(inputs=x), is_training=True, drop_output_collections=())
    (out.square().mean() + oc.module_outputs["aux_loss"]).backward()
    for name in ("gate_weight", "wi_0_weight", "wi_1_weight", "wo_weight"):
        assert params[name].grad is not None and params[name].grad.abs().sum() > 0, name
    assert x.grad.abs().sum() > 0


def test_bias_gating_updates_bias_towards_underused_experts():
    layer, params = _layer(gating=TopKBiasGating.default_config().set(gating_update_rate=0.1))
    assert params["gating"]["gate_bias"].shape == (4,)
    x = torch.randn(2, 16, 16)
    _, oc = functional(layer, prng.PRNGKey(1), params, dict(inputs=x), is_training=True, drop_output_collections=())
    new_bias = oc.state_updates["gating"]["gate_bias"]
    assignment = oc.module_outputs["gating"]["gate_assignment"]
    counts = torch.bincount(assignment.reshape(-1), minlength=4).float()
    expect = 0.1 * torch.sign(counts.mean() - counts)
    torch.testing.assert_close(new_bias, expect)


def test_convert_dense_to_moe():
    dense = {"linear1_0": {"weight": torch.randn(8, 16)}, "linear1_1": {"weight": torch.randn(8, 16)},
             "linear2": {"weight": torch.randn(16, 8)}, "norm": {"scale": torch.ones(8)}}
    moe = convert_dense_to_moe_parameters(dense, num_experts=3, activation=("nn.silu", "linear"))
    assert moe["wi_0_weight"].shape == (3, 8, 16) and moe["wo_weight"].shape == (3, 16, 8)
    assert moe["gate_weight"].shape == (8, 3)
    torch.testing.assert_close(moe["wi_1_weight"][2], dense["linear1_1"]["weight"])


@pytest.mark.gpu
@pytest.mark.parametrize("num_experts,k_dim,n_dim", [(4, 256, 512), (8, 128, 192), (3, 512, 64), (8, 1024, 640)])
def test_grouped_linear_kernel_matches_reference(num_experts, k_dim, n_dim):
    from axlearn_b200.ops import cuda_ops

    torch.manual_seed(2)
    experts = torch.randint(0, num_experts, (2, 900), device="cuda")
    experts[experts == 1] = 0                      # an empty expert
    dest, offsets, block_expert, rows = moe_ops.padded_group_layout(experts, num_experts)
    src = torch.randn(experts.numel(), k_dim, device="cuda").bfloat16()
    x = torch.zeros(rows, k_dim, device="cuda", dtype=torch.bfloat16)
    x[dest.long()] = src
    w = (torch.randn(num_experts, k_dim, n_dim, device="cuda") / k_dim ** 0.5).bfloat16()
    xg, wg = x.clone().requires_grad_(), w.clone().requires_grad_()
    y = moe_ops.grouped_linear(xg, wg, offsets, block_expert)
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    yr = moe_ops.grouped_linear_reference(xr, wr, offsets)
    used = int(offsets[-1])
    scale = yr.abs().max().item()
    assert (y[:used].float() - yr[:used]).abs().max().item() < 2e-2 * scale
    g = torch.zeros_like(yr)
    g[dest.long()] = torch.randn(experts.numel(), n_dim, device="cuda")
    g = g.bfloat16()
    y.backward(g)
    yr.backward(g.float())
    torch.cuda.synchronize()
    cuda_ops.check_status()
    assert (xg.grad[:used].float() - xr.grad[:used]).abs().max().item() < 2e-2 * xr.grad.abs().max().item()
    assert (wg.grad.float() - wr.grad).abs().max().item() < 2e-2 * wr.grad.abs().max().item()
    assert wg.grad[1].abs().max().item() == 0      # the empty expert gets a zero gradient


@pytest.mark.gpu
def test_dropfree_layer_on_gpu_matches_cpu():
    layer, params = _layer(num_experts=4, k=2, dim=128, hidden=256)
    torch.manual_seed(3)
    x = torch.randn(2, 96, 128).bfloat16().float()
    # The oracle sees the same bf16-rounded values; a token whose two best router scores are
    # nearly tied may still pick another expert under bf16 arithmetic, so a few outliers pass.
    rounded = {k: (v.bfloat16().float() if torch.is_tensor(v) else {kk: vv.bfloat16().float() for kk, vv in v.items()})
               for k, v in params.items()}
    ref, _ = functional(layer, prng.PRNGKey(1), rounded, dict(inputs=x), is_training=True, drop_output_collections=())
    to_gpu = lambda t: t.cuda().bfloat16()
    gpu_params = {k: (to_gpu(v) if torch.is_tensor(v) else {kk: to_gpu(vv) for kk, vv in v.items()})
                  for k, v in params.items()}
    out, _ = functional(layer, prng.PRNGKey(1), gpu_params, dict(inputs=to_gpu(x)), is_training=True, drop_output_collections=())
    err = (out.float().cpu() - ref).abs().amax(dim=-1).reshape(-1)
    scale = ref.abs().max().item()
    assert (err < 5e-2 * scale).float().mean().item() > 0.9, err
    assert err.median().item() < 2e-2 * scale, err


def _train_qwen(directory, steps, device="cpu"):
    from axlearn_b200.experiments.text.gpt import qwen
    from axlearn_b200.experiments.text.gpt.common import (
        adamw_decoupled_learner_config,
        get_trainer_config_fn,
        mesh_shape_from_axes,
    )

    model = qwen.preset("test")
    learner = adamw_decoupled_learner_config(peak_lr=3e-3, max_step=steps, weight_decay=1e-4, lr_warmup_steps=1)
    cfg = get_trainer_config_fn(
        model_cfg=model, learner_cfg=learner, max_step=steps, train_batch_size=4, max_sequence_length=32,
        vocab_size=512, mesh_shape=mesh_shape_from_axes(), save_every_n_steps=1000)()
    cfg.dir = str(directory)
    cfg.device = device
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    data = iter(trainer.input.dataset())
    batch = next(data)
    return trainer, [trainer.train_step(batch)["loss"].item() for _ in range(steps)]


def test_qwen3_style_model_trains(tmp_path):
    """Tiny Qwen3-style model (drop-free experts, decoupled attention width, QK norm): the loss on
    a repeated batch goes down and the per-layer parameters have the expected shapes."""
    trainer, losses = _train_qwen(tmp_path, 8)
    assert losses[-1] < losses[0] - 0.2, losses
    layer = trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]
    assert layer["feed_forward"]["wi_0_weight"].shape == (2, 8, 64, 64)
    assert layer["self_attention"]["attention"]["o_proj"]["weight"].shape[-2:] == (4, 32)
    assert "norm" in layer["self_attention"]["attention"]["scale_query"]


@pytest.mark.gpu
def test_qwen3_style_model_trains_on_gpu(tmp_path):
    _, cpu_losses = _train_qwen(tmp_path / "cpu", 3)
    _, gpu_losses = _train_qwen(tmp_path / "gpu", 3, device="cuda")
    for a, b in zip(cpu_losses, gpu_losses):
        assert abs(a - b) < 0.05 * abs(a), (cpu_losses, gpu_losses)


def test_approximate_dropfree_matches_dropfree_when_nothing_is_dropped():
    from axlearn_b200.common.mixture_of_experts import ApproximateTokenDropFreeMoE

    layer, params = _layer()
    cfg = ApproximateTokenDropFreeMoE.default_config().set(
        name="moe", input_dim=16, hidden_dim=32, num_experts=4, num_groups=1, activation=("nn.silu", "linear"),
        structure="prenorm", expert_parallel_capacity=4.0)        # room for every assignment
    cfg.gating.set(num_experts_per_token=2)
    approx = cfg.instantiate(parent=None)
    torch.manual_seed(5)
    x = torch.randn(2, 12, 16)
    want, _ = functional(layer, prng.PRNGKey(1), params, dict(inputs=x), is_training=True, drop_output_collections=())
    got, oc = functional(approx, prng.PRNGKey(1), params, dict(inputs=x), is_training=True, drop_output_collections=())
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    assert float(oc.summaries["dropped_token_ratio"]) == 0.0
    # A tight buffer drops the overflow and says so.
    tight = cfg.clone(expert_parallel_capacity=0.5).instantiate(parent=None)
    _, oc2 = functional(tight, prng.PRNGKey(1), params, dict(inputs=x), is_training=True, drop_output_collections=())
    assert float(oc2.summaries["dropped_token_ratio"]) > 0.3
