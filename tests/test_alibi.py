"""ALiBi and the other attention logit-bias layers; a decoder with ``attention_mask``."""
import torch

from axlearn_b200.common import attention_logit_bias as alb
from axlearn_b200.common import prng
from axlearn_b200.common.decoder import Decoder
from axlearn_b200.common.module import functional


def test_slopes():
    assert alb.alibi_get_slopes(8) == [2 ** -(i + 1) for i in range(8)]
    s12 = alb.alibi_get_slopes(12)
    assert s12[:8] == alb.alibi_get_slopes(8) and s12[8:] == alb.alibi_get_slopes(16)[0::2][:4]


def test_alibi_bias_values_and_segments():
    layer = alb.ALiBiAttentionLogitBiasLayer.default_config().set(name="a", num_heads=4).instantiate(parent=None)
    seg = torch.tensor([[1, 1, 1, 2, 2]])
    pos = torch.tensor([[0, 1, 2, 0, 1]])
    bias, _ = functional(layer, None, {}, dict(segment_ids=seg, positions=pos), is_training=False)
    assert bias.shape == (1, 4, 5, 5)
    slopes = alb.alibi_get_slopes(4)
    assert bias[0, 1, 2, 0] == -2 * slopes[1] and bias[0, 1, 2, 2] == 0
    assert bias[0, 0, 0, 1] <= alb.NEG_INF / 2 and bias[0, 0, 3, 1] <= alb.NEG_INF / 2     # future; other segment
    assert bias[0, 3, 4, 3] == -slopes[3]
    sym = alb.SymmetricALiBiAttentionLogitBiasLayer.default_config().set(name="s", num_heads=4).instantiate(parent=None)
    b2, _ = functional(sym, None, {}, dict(segment_ids=torch.ones(1, 4, dtype=torch.long), positions=torch.arange(4)[None]),
                       is_training=False)
    torch.testing.assert_close(b2, b2.transpose(-1, -2))
    assert b2[0, 2, 0, 3] == -3 * slopes[2]


def test_decoder_with_alibi_decodes_like_it_trains():
    cfg = Decoder.default_config().set(name="dec", vocab_size=40, dim=16)
    cfg.transformer.num_layers = 2
    cfg.transformer.layer.self_attention.attention.num_heads = 4
    cfg.transformer.layer.feed_forward.hidden_dim = 32
    cfg.attention_mask = alb.ALiBiAttentionLogitBiasLayer.default_config().set(num_heads=4)
    dec = cfg.instantiate(parent=None)
    params = dec.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    ids = torch.randint(1, 40, (2, 7))
    out, _ = functional(dec, None, params, dict(input_batch={"input_ids": ids}), is_training=False)
    full = out["hidden_states"]
    # Position matters although there is no positional embedding: swapping two earlier tokens
    # changes the last position's output.
    swapped = ids.clone()
    swapped[:, [0, 3]] = ids[:, [3, 0]]
    out2, _ = functional(dec, None, params, dict(input_batch={"input_ids": swapped}), is_training=False)
    assert not torch.allclose(out2["hidden_states"][:, -1], full[:, -1], atol=1e-4)
    # Prefill 4 tokens, then extend one token at a time: same hidden states as the full forward.
    padded = torch.zeros(2, 10, dtype=ids.dtype)
    padded[:, :4] = ids[:, :4]
    (states, pre), _ = functional(dec, None, params, dict(
        time_step=torch.full((2,), 4, dtype=torch.int32), input_batch={"input_ids": padded}, max_sequence_length=10),
        is_training=False, method="prefill_states")
    torch.testing.assert_close(pre["hidden_states"][:, :4], full[:, :4], rtol=1e-4, atol=1e-5)
    for t in range(4, 7):
        (states, step), _ = functional(dec, None, params, dict(cached_states=states, input_ids=ids[:, t:t + 1]),
                                       is_training=False, method="extend_step")
        torch.testing.assert_close(step["hidden_states"][:, 0], full[:, t], rtol=1e-4, atol=1e-5)
