"""T5 relative position buckets (against transformers) and the T5-style encoder."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.common.t5 import T5RelativePositionalEmbedding, t5_encoder_config, t5_relative_position_bucket
from axlearn_b200.common.utils import flatten_items


@pytest.mark.parametrize("bidirectional", [True, False])
def test_buckets_match_transformers(bidirectional):
    t5 = pytest.importorskip("transformers.models.t5.modeling_t5")
    rel = torch.arange(-300, 300)[None, :] - torch.zeros(1, 1, dtype=torch.long)
    want = t5.T5Attention._relative_position_bucket(rel, bidirectional=bidirectional, num_buckets=32, max_distance=128)
    got = t5_relative_position_bucket(rel, bidirectional=bidirectional, num_buckets=32, max_distance=128)
    assert torch.equal(got, want)


def test_relative_bias_layer_and_encoder():
    layer = T5RelativePositionalEmbedding.default_config().set(name="rel", dim=4, num_buckets=8,
                                                               max_distance=16).instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    bias, _ = functional(layer, prng.PRNGKey(1), params, dict(query_len=5, key_len=7), is_training=False)
    assert bias.shape == (1, 4, 5, 7)
    # Toeplitz: the bias depends on key - query only.
    torch.testing.assert_close(bias[0, :, 1, 2], bias[0, :, 3, 4])
    cfg = t5_encoder_config(vocab_size=50, dim=32, num_layers=2, num_attention_heads=4, ffn_dim=64).set(name="enc")
    enc = cfg.instantiate(parent=None)
    p = enc.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    names = [n for n, _ in flatten_items(p)]
    assert not any(n.endswith("/bias") for n in names)                      # T5 has no biases
    assert "relative_pos_emb/emb/weight" in names and "output/norm/scale" in names and not any("pos_emb/weight" == n for n in names)
    ids = torch.randint(1, 50, (2, 9))
    ids[1, 6:] = 0
    out, _ = functional(enc, prng.PRNGKey(1), p, dict(input_ids=ids), is_training=False)
    assert out.shape == (2, 9, 32)
    # Padded keys are invisible: changing the padded tail's ids leaves live positions unchanged.
    ids2 = ids.clone()
    out2, _ = functional(enc, prng.PRNGKey(1), p, dict(input_ids=ids2), is_training=False)
    torch.testing.assert_close(out2[1, :6], out[1, :6])
    # Causal variant: position t does not depend on later tokens.
    dec = t5_encoder_config(vocab_size=50, dim=32, num_layers=1, num_attention_heads=4, causal=True).set(name="dec").instantiate(parent=None)
    pd = dec.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    a = torch.randint(1, 50, (1, 8))
    b = a.clone()
    b[0, 5:] = torch.randint(1, 50, (3,))
    oa, _ = functional(dec, prng.PRNGKey(1), pd, dict(input_ids=a), is_training=False)
    ob, _ = functional(dec, prng.PRNGKey(1), pd, dict(input_ids=b), is_training=False)
    torch.testing.assert_close(oa[0, :5], ob[0, :5])
