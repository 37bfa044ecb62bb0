"""YaRN RoPE scaling: parameters against transformers, and use inside the attention projections."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.attention import (
    FusedQKVLinear,
    RoFormerQKVLinear,
    RoFormerSinusoidalPositionalEmbedding,
    YaRNSinusoidalPositionalEmbedding,
)
from axlearn_b200.common.module import functional


def _yarn(**kw):
    cfg = YaRNSinusoidalPositionalEmbedding.default_config().set(
        name="yarn", dim=64, theta=10000.0, original_max_seq_length=2048, scaling_factor=4.0, **kw)
    return cfg.instantiate(parent=None)


def test_parameters_match_transformers():
    rope_utils = pytest.importorskip("transformers.modeling_rope_utils")
    transformers = pytest.importorskip("transformers")
    hf_cfg = transformers.LlamaConfig(
        hidden_size=64 * 4, num_attention_heads=4, max_position_embeddings=8192, rope_theta=10000.0,
        rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 2048,
                      "beta_fast": 32.0, "beta_slow": 1.0})
    try:
        inv_freq, attention_factor = rope_utils.ROPE_INIT_FUNCTIONS["yarn"](hf_cfg, "cpu")
    except Exception as e:  # pylint: disable=broad-except
        pytest.skip(f"transformers' yarn initialiser has another signature here: {e}")
    ours_inv, ours_scale = _yarn().compute_rope_params()
    torch.testing.assert_close(ours_inv, inv_freq.float(), rtol=1e-5, atol=1e-8)
    assert ours_scale == pytest.approx(float(attention_factor), rel=1e-6)


def test_yarn_limits_and_projection_path():
    # scaling_factor 1 is plain RoPE.
    plain = RoFormerSinusoidalPositionalEmbedding.default_config().set(name="p", dim=64).instantiate(parent=None)
    same = YaRNSinusoidalPositionalEmbedding.default_config().set(
        name="y", dim=64, original_max_seq_length=2048, scaling_factor=1.0).instantiate(parent=None)
    pos = torch.arange(50)[None]
    a, _ = functional(plain, None, {}, dict(positions=pos), is_training=False)
    b, _ = functional(same, None, {}, dict(positions=pos), is_training=False)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    # With scaling the fastest dimension is untouched and the slowest is interpolated by the factor.
    inv, scale = _yarn().compute_rope_params()
    base = 1.0 / 10000.0 ** (2 * torch.arange(32) / 64)
    assert inv[0].item() == pytest.approx(base[0].item()) and inv[-1].item() == pytest.approx(base[-1].item() / 4, rel=1e-5)
    assert scale > 1.0
    # Inside the projection: q / k rotated with the scaled table; relative-position property holds.
    cfg = RoFormerQKVLinear.default_config().set(
        name="qkv", query_dim=32, key_dim=32, value_dim=32, num_heads=2, per_head_dim=16,
        input_linear=FusedQKVLinear.default_config(), rotary_value=False,
        rope_pos_emb_layer=YaRNSinusoidalPositionalEmbedding.default_config().set(
            original_max_seq_length=8, scaling_factor=2.0))
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    x = torch.randn(1, 6, 32)
    out0, _ = functional(layer, None, params, dict(query=x, query_positions=torch.arange(6)[None]), is_training=False)
    out5, _ = functional(layer, None, params, dict(query=x, query_positions=torch.arange(6)[None] + 5), is_training=False)
    s0 = torch.einsum("btnh,bsnh->bnts", out0.query, out0.key)
    s5 = torch.einsum("btnh,bsnh->bnts", out5.query, out5.key)
    torch.testing.assert_close(s0, s5, rtol=1e-4, atol=1e-4)          # logits depend on t - s only
    torch.testing.assert_close(out0.value, out5.value)
    assert not torch.allclose(out0.query, out5.query)
