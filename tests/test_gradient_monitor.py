"""Activation-gradient monitor: clipping in the backward pass and statistics as pseudo-gradients."""
import torch

from axlearn_b200.common import gradient_monitor as gm
from axlearn_b200.common import learner as learner_lib
from axlearn_b200.common import optimizers, prng
from axlearn_b200.common.attention import TransformerFeedForwardLayer
from axlearn_b200.common.base_layer import ParameterSpec
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.module import functional
from axlearn_b200.common.utils import flatten_items, tree_map


def test_top_k_clip_zeroes_the_largest_tokens_and_reports_their_norms():
    g = torch.randn(2, 8, 16)
    g[0, 3] *= 50
    g[1, 5] *= 30
    for method in ("approx", "topk", "sort"):
        clipped, stats = gm.top_k_clip_fn(k=2, method=method)(g)
        norms = g.norm(dim=-1).reshape(-1)
        top = norms.topk(2).values
        torch.testing.assert_close(stats, top)
        if method == "approx":
            assert clipped[0, 3].abs().sum() == 0 and clipped[1, 5].abs().sum() == 0
            assert (clipped.reshape(16, 16).abs().sum(-1) == 0).sum() == 2
        else:  # everything at or above the k-th norm goes: the k-th itself included
            assert clipped[0, 3].abs().sum() == 0 and clipped[1, 5].abs().sum() == 0
        kept = clipped.reshape(16, 16)[[0, 1, 2]]
        torch.testing.assert_close(kept, g.reshape(16, 16)[[0, 1, 2]])


def test_positions_survive_the_bf16_byte_encoding():
    ids = torch.tensor([0, 255, 256, 70000, 2 ** 31 - 1], dtype=torch.int32)
    enc = gm.encode_int32_to_bf16_bytes(ids)
    assert enc.dtype == torch.bfloat16 and enc.shape == (4, 5)
    assert torch.equal(gm.decode_bf16_bytes_to_int32(enc), ids)
    _, stats = gm.top_k_clip_fn(k=3, log_pos=True)(torch.randn(4, 100, 8))
    assert stats.shape == (5, 3)


def test_percentile_fn_leaves_the_gradient_alone():
    g = torch.randn(4, 64, 8)
    out, stats = gm.compute_grad_percentile_no_clip_fn((50, 99))(g)
    assert out is g
    torch.testing.assert_close(stats[0], g.norm(dim=-1).reshape(-1).median(), rtol=0.05, atol=0.05)


def test_monitored_ffn_clips_parameter_gradients_and_the_stats_reach_the_summaries():
    base = TransformerFeedForwardLayer.default_config().set(input_dim=8, hidden_dim=16)
    cfg = gm.convert_to_monitored_layer_config(base)
    cfg.gradient_monitor.set(stats_shape=(2,))
    cfg.gradient_monitor.clip_fn.set(k=2, method="topk")
    layer = cfg.set(name="ffn").instantiate(parent=None)
    assert type(layer).__name__ == "MonitoredTransformerFeedForwardLayer"
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert params["gradient_monitor"]["stats"].shape == (2,)
    plain = base.set(name="ffn").instantiate(parent=None)
    plain_params = {k: v for k, v in params.items() if k != "gradient_monitor"}

    x = torch.randn(2, 6, 8)
    w = torch.ones(2, 6, 1)
    w[0, 1] = 100.0   # two tokens dominate dL/dy
    w[1, 4] = 60.0

    def grads(mod, prm, weight):
        prm = tree_map(lambda t: t.clone().requires_grad_(True), prm)
        y, col = functional(mod, prng.PRNGKey(1), prm, [x], is_training=True, drop_output_collections=())
        (y * weight).sum().backward()
        return {p: t.grad for p, t in flatten_items(prm)}, col

    monitored, _ = grads(layer, params, w)
    w_clipped = w.clone()
    w_clipped[0, 1] = 0
    w_clipped[1, 4] = 0
    expected, _ = grads(plain, plain_params, w_clipped)
    for p, g in expected.items():
        torch.testing.assert_close(monitored[p], g, rtol=1e-5, atol=1e-6)
    stats = monitored["gradient_monitor/stats"]
    torch.testing.assert_close(stats, torch.tensor([100.0, 60.0]) * 8 ** 0.5)

    # The stats parameter takes its "gradient" as its value through the composite learner.
    inner = learner_lib.Learner.default_config().set(
        optimizer=config_for_function(optimizers.sgd_optimizer).set(learning_rate=0.1, decouple_weight_decay=False))
    lcfg = gm.gradient_monitoring_learner_cfg_modifier(inner)
    lrn = lcfg.set(name="learner").instantiate(parent=None)
    specs = tree_map(lambda t: ParameterSpec(shape=tuple(t.shape), mesh_axes=(None,) * t.ndim), params)
    opt_params = tree_map(lambda t: optimizers.OptParam(t, None, None), params)
    state = lrn.init(opt_params)
    from axlearn_b200.common.utils import unflatten_items
    lrn.update(model_params=params, gradients=unflatten_items(list(monitored.items())), state=state, param_specs=specs)
    torch.testing.assert_close(params["gradient_monitor"]["stats"], stats)
    _, col = grads(layer, params, w)
    logged = dict(flatten_items(col.summaries))
    key = [k for k in logged if k.endswith("top_norms_hist")]
    assert key, logged.keys()
