"""DeBERTa v2 against the Hugging Face implementation; DistilBERT encoder config."""
import pytest
import torch

from axlearn_b200.common import deberta as db
from axlearn_b200.common import prng
from axlearn_b200.common.attention import StackedTransformerLayer
from axlearn_b200.common.distilbert import set_distilbert_config
from axlearn_b200.common.module import functional
from axlearn_b200.common.text_encoder import TEXT_EMBEDDINGS
from axlearn_b200.common.utils import flatten_items


def test_log_buckets():
    b = db.deberta_relative_position_bucket(query_len=12, key_len=12, num_directional_buckets=4, max_distance=16)
    assert b.shape == (12, 12) and b.min() >= 0 and b.max() <= 8
    assert torch.equal(b.diagonal(), torch.full((12,), 4))
    assert b[2, 0] == 6 and b[0, 2] == 2                       # small distances keep their own bucket
    assert torch.equal(b + b.t(), torch.full((12, 12), 8))     # antisymmetric around the centre
    assert (b[:, 0].diff() >= 0).all()


def _encoder(attention_type):
    cfg = db.deberta_v2_encoder_config(dim=16, vocab_size=50, num_layers=2, max_distance=8,
                                       num_directional_buckets=4, stack_cls=StackedTransformerLayer)
    cfg.transformer.layer.self_attention.attention = db.deberta_v2_self_attention_config(
        num_heads=2, max_distance=8, num_directional_buckets=4, hidden_dropout=0, attention_dropout=0,
        attention_type=attention_type, base_cfg=cfg.transformer.layer.self_attention.attention)
    cfg.transformer.layer.feed_forward.activation = "exact_gelu"
    return cfg.set(name="enc", pad_token_id=0).instantiate(parent=None)


@pytest.mark.parametrize("types", [("p2c", "c2p"), ("c2p",), ("p2c",)])
def test_matches_hugging_face_deberta_v2(types):
    transformers = pytest.importorskip("transformers")
    hf_cfg = transformers.DebertaV2Config(
        vocab_size=50, hidden_size=16, num_hidden_layers=2, num_attention_heads=2, intermediate_size=64,
        hidden_act="gelu", hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, max_position_embeddings=32,
        type_vocab_size=0, relative_attention=True, max_relative_positions=8, position_buckets=4,
        pos_att_type=list(types), share_att_key=True, norm_rel_ebd="layer_norm", position_biased_input=False,
        layer_norm_eps=1e-7, pad_token_id=0)
    torch.manual_seed(0)
    hf = transformers.DebertaV2Model(hf_cfg).eval()
    for p in hf.parameters():                                   # biases and norms away from their defaults
        torch.nn.init.normal_(p, std=0.2)
    sd = hf.state_dict()
    enc = _encoder(tuple(db.DisentangledAttentionType[t.upper()] for t in types))
    params = enc.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")

    def put(path, value):
        node = params
        *head, last = path.split("/")
        for k in head:
            node = node[k]
        assert node[last].shape == value.shape, (path, node[last].shape, value.shape)
        node[last] = value.clone()

    put("emb/token_emb/weight", sd["embeddings.word_embeddings.weight"])
    put("emb/norm/scale", sd["embeddings.LayerNorm.weight"])
    put("emb/norm/bias", sd["embeddings.LayerNorm.bias"])
    put("relative_pos_emb/weight", sd["encoder.rel_embeddings.weight"])
    put("relative_pos_emb/norm/scale", sd["encoder.LayerNorm.weight"])
    put("relative_pos_emb/norm/bias", sd["encoder.LayerNorm.bias"])
    for i in range(2):
        src, dst = f"encoder.layer.{i}.", f"transformer/layer{i}/"
        for ours, theirs in (("q_proj", "query_proj"), ("k_proj", "key_proj"), ("v_proj", "value_proj")):
            put(dst + f"self_attention/attention/i_proj/{ours}/weight",
                sd[src + f"attention.self.{theirs}.weight"].t().reshape(16, 2, 8))
            put(dst + f"self_attention/attention/i_proj/{ours}/bias", sd[src + f"attention.self.{theirs}.bias"].reshape(2, 8))
        put(dst + "self_attention/attention/o_proj/weight", sd[src + "attention.output.dense.weight"].reshape(16, 2, 8))
        put(dst + "self_attention/attention/o_proj/bias", sd[src + "attention.output.dense.bias"])
        put(dst + "self_attention/norm/scale", sd[src + "attention.output.LayerNorm.weight"])
        put(dst + "self_attention/norm/bias", sd[src + "attention.output.LayerNorm.bias"])
        put(dst + "feed_forward/linear1/weight", sd[src + "intermediate.dense.weight"].t())
        put(dst + "feed_forward/linear1/bias", sd[src + "intermediate.dense.bias"])
        put(dst + "feed_forward/linear2/weight", sd[src + "output.dense.weight"].t())
        put(dst + "feed_forward/linear2/bias", sd[src + "output.dense.bias"])
        put(dst + "feed_forward/norm/scale", sd[src + "output.LayerNorm.weight"])
        put(dst + "feed_forward/norm/bias", sd[src + "output.LayerNorm.bias"])

    ids = torch.tensor([[5, 7, 9, 11, 13, 2, 0, 0], [3, 4, 6, 8, 10, 12, 14, 16]])
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=(ids != 0).long()).last_hidden_state
    got, _ = functional(enc, None, params, dict(input_ids=ids), is_training=False)
    live = ids != 0
    torch.testing.assert_close(got[live], want[live], rtol=2e-4, atol=2e-4)


def test_deberta_model_config_builds_and_trains_one_step():
    enc = db.deberta_v2_encoder_config(dim=16, vocab_size=50, num_layers=2, max_distance=8)
    enc.transformer.layer.self_attention.attention = db.deberta_v2_self_attention_config(
        num_heads=2, max_distance=8, base_cfg=enc.transformer.layer.self_attention.attention)
    model = db.deberta_v2_model_config(encoder_cfg=enc).set(name="m").instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    names = [k for k, _ in flatten_items(params)]
    assert any("relative_pos_emb/weight" in n for n in names)
    assert not any("pos_q_proj" in n or "pos_k_proj" in n for n in names)     # shared projections
    ids = torch.randint(1, 50, (2, 6))
    batch = dict(input_ids=ids, target_labels=torch.where(torch.rand(2, 6) < 0.5, ids, torch.full_like(ids, -100)))
    out, _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=True)
    loss = out[0] if isinstance(out, tuple) else out
    assert torch.isfinite(loss)


def test_distilbert_config():
    cfg = set_distilbert_config(vocab_size=40, num_layers=2, model_dim=16, num_heads=2, max_seq_len=10)
    assert cfg.encoder.transformer.layer.self_attention.dropout.rate == 0.1
    layer = cfg.set(name="d").instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert "type_emb" not in params["encoder"]["emb"]
    out, _ = functional(layer, None, params, [torch.randint(1, 40, (3, 7))], is_training=False)
    assert out[TEXT_EMBEDDINGS].shape == (3, 1, 16)
