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


def test_t5_encoder_decoder_matches_hugging_face_and_decodes_incrementally():
    import pytest

    transformers = pytest.importorskip("transformers")
    from axlearn_b200.common import prng, t5
    from axlearn_b200.common.module import functional
    from axlearn_b200.common.param_converter import t5_hf_to_encoder_decoder

    hf_cfg = transformers.T5Config(
        vocab_size=50, d_model=16, d_kv=8, d_ff=32, num_layers=2, num_decoder_layers=2, num_heads=2,
        relative_attention_num_buckets=32, relative_attention_max_distance=128, dropout_rate=0.0,
        feed_forward_proj="gated-gelu", tie_word_embeddings=False, layer_norm_epsilon=1e-6, decoder_start_token_id=0)
    torch.manual_seed(0)
    hf = transformers.T5ForConditionalGeneration(hf_cfg).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.3)
    cfg = t5.t5_encoder_decoder_config(vocab_size=50, dim=16, num_attention_heads=2, num_encoder_layers=2,
                                       num_decoder_layers=2, ffn_dim=32).set(name="t5")
    model = cfg.instantiate(parent=None)
    params = t5_hf_to_encoder_decoder(hf.state_dict(), num_heads=2, num_encoder_layers=2, num_decoder_layers=2)
    want_tree = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    from axlearn_b200.common.utils import flatten_items
    assert {k: tuple(v.shape) for k, v in flatten_items(params)} == {k: tuple(v.shape) for k, v in flatten_items(want_tree)}
    src = torch.tensor([[5, 6, 7, 8, 9, 1, 0, 0], [11, 12, 13, 14, 15, 16, 17, 1]])
    tgt = torch.tensor([[0, 21, 22, 23, 1], [0, 31, 32, 1, 0]])
    with torch.no_grad():
        want = hf(input_ids=src, attention_mask=(src != 0).long(), decoder_input_ids=tgt).logits
    batch = {"source": {"input_ids": src}, "target": {"input_ids": tgt}, "target_labels": tgt}
    out, _ = functional(model, None, params, dict(input_batch=batch), is_training=False, method="predict")
    torch.testing.assert_close(out["logits"], want, rtol=2e-3, atol=2e-3)
    # Incremental decoding through the decoder's attention-mask layer gives the same logits.
    dec = model.decoder
    enc = out["encoder_output"]
    cross_bias = torch.where((src != 0)[:, None, None, :], 0.0, -1e9)
    padded = torch.zeros(2, 6, dtype=tgt.dtype)
    padded[:, :2] = tgt[:, :2]
    (states, _), _ = functional(dec, None, params["decoder"], dict(
        time_step=torch.full((2,), 2, dtype=torch.int32), input_batch={"input_ids": padded}, max_sequence_length=6,
        cross_attention_data=enc, cross_attention_logit_biases=cross_bias), is_training=False, method="prefill_states")
    for t in range(2, 4):
        (states, step), _ = functional(dec, None, params["decoder"], dict(
            cached_states=states, input_ids=tgt[:, t:t + 1], cross_attention_data=enc,
            cross_attention_logit_biases=cross_bias), is_training=False, method="extend_step")
        torch.testing.assert_close(step["logits"][:, 0], want[:, t], rtol=2e-3, atol=2e-3)


def test_t5x_tree_converts_to_the_same_parameters_as_hugging_face():
    """A T5X-layout tree built from a Hugging Face model's weights must convert to exactly the
    parameters the Hugging Face converter gives (which is checked against ``transformers`` above)."""
    import numpy as np
    import pytest

    transformers = pytest.importorskip("transformers")
    from axlearn_b200.common.param_converter import t5_hf_to_encoder_decoder
    from axlearn_b200.common.t5x_param_converter import parameters_from_t5x_encoder_decoder, t5x_to_hf_state_dict
    from axlearn_b200.common.utils import flatten_items

    hf_cfg = transformers.T5Config(vocab_size=40, d_model=16, d_kv=8, d_ff=24, num_layers=2, num_decoder_layers=3,
                                   num_heads=2, feed_forward_proj="gated-gelu", tie_word_embeddings=False)
    torch.manual_seed(1)
    sd = transformers.T5ForConditionalGeneration(hf_cfg).state_dict()

    def kernel(key):                    # HF Linear weight [out, in] -> T5X kernel [in, out], as numpy
        return sd[key].t().contiguous().numpy()

    def attention(prefix):
        return {name: {"kernel": kernel(prefix + short + ".weight")}
                for name, short in (("query", "q"), ("key", "k"), ("value", "v"), ("out", "o"))}

    def mlp(prefix):
        return {n: {"kernel": kernel(prefix + n + ".weight")} for n in ("wi_0", "wi_1", "wo")}

    rel = "block.0.layer.0.SelfAttention.relative_attention_bias.weight"
    t5x = {"token_embedder": {"embedding": sd["shared.weight"].numpy()},
           "encoder": {"relpos_bias": {"rel_embedding": sd["encoder." + rel].t().numpy()},
                       "encoder_norm": {"scale": sd["encoder.final_layer_norm.weight"].numpy()}},
           "decoder": {"relpos_bias": {"rel_embedding": sd["decoder." + rel].t().numpy()},
                       "decoder_norm": {"scale": sd["decoder.final_layer_norm.weight"].numpy()},
                       "logits_dense": {"kernel": kernel("lm_head.weight")}}}
    for i in range(2):
        p = f"encoder.block.{i}.layer."
        t5x["encoder"][f"layers_{i}"] = {
            "attention": attention(p + "0.SelfAttention."), "pre_attention_layer_norm": {"scale": sd[p + "0.layer_norm.weight"].numpy()},
            "mlp": mlp(p + "1.DenseReluDense."), "pre_mlp_layer_norm": {"scale": sd[p + "1.layer_norm.weight"].numpy()}}
    for i in range(3):
        p = f"decoder.block.{i}.layer."
        t5x["decoder"][f"layers_{i}"] = {
            "self_attention": attention(p + "0.SelfAttention."),
            "pre_self_attention_layer_norm": {"scale": sd[p + "0.layer_norm.weight"].numpy()},
            "encoder_decoder_attention": attention(p + "1.EncDecAttention."),
            "pre_cross_attention_layer_norm": {"scale": sd[p + "1.layer_norm.weight"].numpy()},
            "mlp": mlp(p + "2.DenseReluDense."), "pre_mlp_layer_norm": {"scale": sd[p + "2.layer_norm.weight"].numpy()}}
    got = parameters_from_t5x_encoder_decoder(t5x, num_heads=2)
    want = t5_hf_to_encoder_decoder(sd, num_heads=2, num_encoder_layers=2, num_decoder_layers=3)
    got_flat, want_flat = dict(flatten_items(got)), dict(flatten_items(want))
    assert set(got_flat) == set(want_flat)
    for k, v in want_flat.items():
        assert torch.equal(got_flat[k], v), k
    # The query kernels carry the sqrt(head_dim) that T5X folds into their initialisation.
    q = got["encoder"]["transformer"]["layer0"]["self_attention"]["attention"]["i_proj"]["q_proj"]["weight"]
    np.testing.assert_allclose(q.reshape(16, 16).numpy(), t5x["encoder"]["layers_0"]["attention"]["query"]["kernel"] * 8 ** 0.5, rtol=1e-6)
    state_dict, n_enc, n_dec = t5x_to_hf_state_dict(t5x)
    assert (n_enc, n_dec) == (2, 3)
    assert set(state_dict) == {k for k in sd if "embed_tokens" not in k}          # the embedding is stored once, as "shared"
    with pytest.raises(ValueError, match="Unsupported layer"):
        parameters_from_t5x_encoder_decoder({**t5x, "extra": {}}, num_heads=2)
    bad = {**t5x, "encoder": {**t5x["encoder"], "layers_0": {**t5x["encoder"]["layers_0"], "mlp": {"wi": {}}}}}
    with pytest.raises(ValueError, match="Unsupported layer"):
        parameters_from_t5x_encoder_decoder(bad, num_heads=2)
