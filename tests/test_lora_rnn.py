import torch

from axlearn_b200.common import lora, prng, rnn
from axlearn_b200.common.module import functional


def _run(cfg, inputs, **kw):
    layer = cfg.set(name="l").instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0))
    out, _ = functional(layer, prng.PRNGKey(1), params, inputs, is_training=False, **kw)
    return layer, params, out


def test_lora_linear_starts_as_the_base_layer_and_trains_only_through_adapters():
    cfg = lora.LoraLinear.default_config().set(input_dim=8, output_dim=6)
    cfg.adapter.set(rank=2, alpha=4.0)
    x = torch.randn(3, 8)
    layer, params, y = _run(cfg, [x])
    base = x @ params["layer"]["weight"] + params["layer"]["bias"]
    assert torch.allclose(y, base, atol=1e-6)                       # lora_up starts at zero
    assert params["adapter"]["lora_down"]["weight"].shape == (8, 2)
    params["adapter"]["lora_up"]["weight"] = torch.ones(2, 6)
    y2, _ = functional(layer, None, params, [x], is_training=False)
    delta = (x @ params["adapter"]["lora_down"]["weight"]) @ torch.ones(2, 6) * 2.0
    assert torch.allclose(y2, base + delta, atol=1e-5)


def test_lora_fused_qkv_adapts_selected_projections():
    cfg = lora.LoraFusedQKVLinear.default_config().set(query_dim=8, key_dim=8, value_dim=8, num_heads=2, per_head_dim=4)
    cfg.adapter.set(rank=2, alpha=2.0)
    _, params, out = _run(cfg, [torch.randn(2, 5, 8)])
    assert set(params) == {"layer", "adapter_query", "adapter_value"}
    assert out.query.shape == (2, 5, 2, 4) and out.value.shape == (2, 5, 2, 4)


def test_lstm_matches_manual_recurrence_and_stack_runs():
    cfg = rnn.LSTMCell.default_config().set(input_dim=5, hidden_dim=7)
    x = torch.randn(4, 3, 5)                                      # [T, B, D]
    layer, params, y = _run(cfg, [x])
    w, b = params["input_proj"]["weight"], params["input_proj"]["bias"]
    m = torch.zeros(3, 7)
    c = torch.zeros(3, 7)
    for t in range(4):
        i, f, g, o = (torch.cat([x[t], m], -1) @ w + b).chunk(4, -1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        m = torch.sigmoid(o) * torch.tanh(c)
        assert torch.allclose(y[t], m, atol=1e-5)
    stack = rnn.StackedRNNLayer.default_config().set(input_dim=5, layers=[
        rnn.LSTMCell.default_config().set(hidden_dim=6), rnn.LSTMCell.default_config().set(hidden_dim=6, output_dim=4)])
    _, _, ys = _run(stack, [x])
    assert ys.shape == (4, 3, 4)
