"""Residual linear attention: chunked form vs scan, semantics, decode state vs full forward."""
import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.common.rattention import (
    RAttention,
    feature_map,
    residual_linear_attention,
    residual_linear_attention_reference,
)


@pytest.mark.parametrize("feat", ["softmax", "relu"])
@pytest.mark.parametrize("chunk", [4, 7, 64])
def test_chunked_matches_scan(feat, chunk):
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 3, 19, 8), torch.randn(2, 3, 19, 8), torch.randn(2, 3, 19, 5)
    h0 = torch.randn(2, 3, 16, 5)
    want, hw = residual_linear_attention_reference(q, k, v, h0, window_size=3, feat_map=feat)
    got, hg = residual_linear_attention(q, k, v, h0, window_size=3, feat_map=feat, chunk_size=chunk)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(hg, hw, rtol=1e-4, atol=1e-4)


def test_linear_branch_only_sees_tokens_outside_the_window():
    q, k, v = torch.randn(1, 1, 10, 4), torch.randn(1, 1, 10, 4), torch.randn(1, 1, 10, 3)
    h0 = torch.zeros(1, 1, 8, 3)
    out, _ = residual_linear_attention(q, k, v, h0, window_size=2, chunk_size=4)
    assert out[0, 0, :3].abs().sum() == 0                          # nothing is older than the window yet
    manual = sum(feature_map(q[0, 0, 5]) @ feature_map(k[0, 0, s])[:, None] * v[0, 0, s] for s in range(0, 3))
    torch.testing.assert_close(out[0, 0, 5], manual.reshape(-1), rtol=1e-4, atol=1e-5)
    v2 = v.clone()
    v2[0, 0, 3:] += 1.0                                            # inside every query's window or in its future
    out2, _ = residual_linear_attention(q, k, v2, h0, window_size=2, chunk_size=4)
    torch.testing.assert_close(out2[0, 0, :6], out[0, 0, :6])


@pytest.mark.parametrize("use_la", [True, False])
def test_layer_decodes_like_it_trains(use_la):
    cfg = RAttention.default_config().set(name="ra", query_dim=16, num_heads=2, sliding_window_size=3, chunk_size=4,
                                          use_residual_la=use_la, use_qk_scale=use_la)
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    x = torch.randn(2, 11, 16)
    full, _ = functional(layer, None, params, [x], is_training=False)
    assert full.shape == (2, 11, 16)
    states, _ = functional(layer, None, params, dict(batch_size=2), is_training=False, method="init_states")
    assert states["k"].shape == (2, 4, 2, 8) and states["h"].shape == (2, 2, 16, 8)      # constant-size state
    for t in range(11):
        (states, y), _ = functional(layer, None, params, dict(cached_states=states, query=x[:, t:t + 1]),
                                    is_training=False, method="extend_step")
        torch.testing.assert_close(y[:, 0], full[:, t], rtol=1e-4, atol=1e-4)
    if use_la:                                                      # distant tokens still matter
        x2 = x.clone()
        x2[:, 0] += torch.randn(2, 16)
        far, _ = functional(layer, None, params, [x2], is_training=False)
        assert not torch.allclose(far[:, 10], full[:, 10], atol=1e-5)
    else:
        x2 = x.clone()
        x2[:, 0] += torch.randn(2, 16)
        far, _ = functional(layer, None, params, [x2], is_training=False)
        torch.testing.assert_close(far[:, 10], full[:, 10])
