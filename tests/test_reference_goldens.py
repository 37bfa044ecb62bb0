"""Numerics against golden vectors recorded by the reference's own tests (inputs, parameters and
expected outputs; ``tests/testdata/golden_vectors.npz`` holds a subset of the arrays of
axlearn/experiments/testdata/*.npz: rotary embeddings, CTC loss, LayerNorm / Linear / max pooling,
a two-layer GPT-2 checked against Hugging Face, BERT embeddings)."""

import os

import numpy as np
import pytest
import torch

from axlearn_b200.common import causal_lm, prng
from axlearn_b200.common.attention import StackedTransformerLayer, apply_rotary_position_embeddings
from axlearn_b200.common.module import functional

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "testdata", "golden_vectors.npz")


@pytest.fixture(scope="module")
def golden():
    data = np.load(_PATH)
    return {k: torch.from_numpy(np.asarray(data[k])) for k in data.keys()}


def _tree(golden, prefix):
    out = {}
    for k, v in golden.items():
        if k.startswith(prefix):
            node = out
            parts = k[len(prefix):].split("/")
            for p in parts[:-1]:
                node = node.setdefault(p, {})
            node[parts[-1]] = v
    return out


@pytest.mark.parametrize("case", ["b2_nh3_ml10_d32_rkTrue_rvTrue", "b2_nh3_ml10_d32_rkFalse_rvFalse",
                                  "b2_nh4_ml8_d16_rkTrue_rvTrue"])
def test_rotary_embeddings(golden, case):
    g = _tree(golden, f"rope_{case}/")
    q, k, v = apply_rotary_position_embeddings(
        query=g["inputs"]["query"], key=g["inputs"]["key"], value=g["inputs"]["value"],
        sinusoidal_pos=g["inputs"]["sinusoidal_pos"], rotary_key=bool(g["params"]["rotary_key"]),
        rotary_value=bool(g["params"]["rotary_value"]))
    torch.testing.assert_close(q, g["outputs"]["q_proj"], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(k, g["outputs"]["k_proj"], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(v, g["outputs"]["v_proj"], rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
def test_rotary_kernel_matches_reference_vectors(golden):
    """The CUDA RoPE kernel against the same vectors (positions 0..T-1, theta 10000)."""
    from axlearn_b200 import ops

    g = _tree(golden, "rope_b2_nh3_ml10_d32_rkTrue_rvTrue/")
    q = g["inputs"]["query"].cuda().bfloat16()
    out = ops.rope(q, torch.arange(q.shape[1], device="cuda"), 10000.0)
    want = g["outputs"]["q_proj"].cuda()
    assert (out.float() - want).abs().max().item() < 0.05 * want.abs().max().item()


@pytest.mark.parametrize("blank", [0, 1])
def test_ctc_loss(golden, blank):
    from axlearn_b200.audio.asr import CTCDecoderModel

    g = _tree(golden, f"ctc_blank{blank}/")
    logits = g["inputs"]["logits"]
    b, t, v = logits.shape
    paddings = (torch.arange(t)[None] >= g["inputs"]["input_lengths"][:, None]).float()
    labels = g["inputs"]["target_labels"].clone().long()
    labels[torch.arange(labels.shape[1])[None] >= g["inputs"]["target_lengths"][:, None]] = -1
    layer = CTCDecoderModel.default_config().set(name="ctc", input_dim=v, vocab_size=v, blank_id=blank).instantiate(parent=None)
    # Identity head: the golden gives logits directly.
    params = {"lm_head": {"weight": torch.eye(v), "bias": torch.zeros(v)}}
    (_, aux), _ = functional(layer, prng.PRNGKey(0), params,
                             dict(input_batch={"inputs": logits, "paddings": paddings, "target_labels": labels}),
                             is_training=False)
    want = g["outputs"]["per_example_loss"]
    weight = g["inputs"]["per_example_weight"]
    got = aux["per_example_loss"] * aux["per_example_weight"]
    torch.testing.assert_close(got * weight, want * weight, rtol=1e-4, atol=1e-4)


def test_layer_norm_linear_maxpool(golden):
    from axlearn_b200.common.layers import LayerNorm, Linear, MaxPool2D

    g = _tree(golden, "layers_layer_norm_against_torch/")
    ln = LayerNorm.default_config().set(name="ln", input_dim=6).instantiate(parent=None)      # default eps 1e-8
    y, _ = functional(ln, None, g["params"], [g["inputs"]["x"]], is_training=False)
    torch.testing.assert_close(y, g["outputs"]["ref"], rtol=1e-5, atol=1e-5)
    g = _tree(golden, "layers_linear/")
    lin = Linear.default_config().set(name="lin", input_dim=4, output_dim=6).instantiate(parent=None)
    y, _ = functional(lin, None, g["params"], [g["inputs"]["x"]], is_training=False)
    torch.testing.assert_close(y, g["outputs"]["ref"], rtol=1e-5, atol=1e-5)
    g = _tree(golden, "layers_maxpool2d_3x3_S2/")
    pool = MaxPool2D.default_config().set(name="pool", window=(3, 3), strides=(2, 2)).instantiate(parent=None)
    y, _ = functional(pool, None, {}, [g["inputs"]["x"]], is_training=False)
    torch.testing.assert_close(y, g["outputs"]["ref"])


def test_gpt2_logits(golden):
    """Two-layer GPT-2 with the reference's parameter tree reproduces the logits that the
    reference recorded from Hugging Face's GPT-2."""
    g = _tree(golden, "gpt2/")
    decoder_cfg = causal_lm.gpt_decoder_config(
        stack_cfg=StackedTransformerLayer.default_config(), num_layers=2, hidden_dim=16, num_heads=4, vocab_size=24,
        activation_function="nn.gelu", max_position_embeddings=11, layer_norm_epsilon=1e-5, dropout_rate=0.0)
    model = causal_lm.Model.default_config().set(name="gpt2", decoder=decoder_cfg).instantiate(parent=None)
    init = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    from axlearn_b200.common.utils import flatten_items

    assert {p: tuple(t.shape) for p, t in flatten_items(init)} == {p: tuple(t.shape) for p, t in flatten_items(g["params"])}
    logits, _ = functional(model, prng.PRNGKey(1), g["params"], dict(input_batch={"input_ids": g["inputs"]["input_ids"].long()}),
                           is_training=False, method="extract_logits")
    torch.testing.assert_close(logits, g["outputs"]["logits"], rtol=1e-4, atol=1e-5)


def test_bert_embeddings(golden):
    from axlearn_b200.common.embedding import LearnedPositionalEmbedding, TransformerTextEmbeddings
    from axlearn_b200.common.layers import Embedding, LayerNorm

    g = _tree(golden, "bert_emb/")
    cfg = TransformerTextEmbeddings.default_config().set(
        name="emb", dim=12, vocab_size=24, pos_emb=LearnedPositionalEmbedding.default_config().set(shape=(11,)),
        type_emb=Embedding.default_config().set(num_embeddings=1), norm=LayerNorm.default_config().set(eps=1e-12))
    layer = cfg.instantiate(parent=None)
    ids = g["inputs"]["input_ids"].long()
    batch = {"inputs": ids, "token_type_ids": torch.zeros_like(ids), "positions": None}
    out, _ = functional(layer, prng.PRNGKey(0), g["params"], dict(input_batch=batch), is_training=False)
    torch.testing.assert_close(out, g["outputs"]["hidden_states"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("case", ["bert_mlm", "bert_mlm_padded"])
def test_bert_masked_lm(golden, case):
    """BERT (post-norm encoder + MLM head) with the reference's parameter tree reproduces the
    hidden states, logits and loss recorded from Hugging Face's ``BertForMaskedLM``."""
    from axlearn_b200.common import encoder
    from axlearn_b200.common.utils import flatten_items

    g = _tree(golden, case + "/")
    cfg = encoder.bert_model_config(vocab_size=24, hidden_dim=16, num_layers=2, num_heads=4, max_position_embeddings=20,
                                    type_vocab_size=2, layer_norm_epsilon=1e-12).set(name="bert")
    cfg.head.ignored_target_id = -100          # Hugging Face's convention, as in the reference's test
    model = cfg.instantiate(parent=None)
    init = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert {p: tuple(t.shape) for p, t in flatten_items(init)} == {p: tuple(t.shape) for p, t in flatten_items(g["params"])}
    batch = {k: g["inputs"][k].long() for k in ("input_ids", "token_type_ids", "target_labels")}
    (loss, aux), _ = functional(model, prng.PRNGKey(1), g["params"], dict(input_batch=batch, return_aux=True), is_training=False)
    live = (batch["input_ids"] != 0)[..., None]
    torch.testing.assert_close(aux["sequence_output"] * live, g["outputs"]["hidden_states_last"] * live, rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(aux["logits"] * live, g["outputs"]["logits"] * live, rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(loss.double(), g["outputs"]["loss"].double(), rtol=1e-4, atol=1e-5)


def test_hf_bert_encoder(golden):
    from axlearn_b200.common import encoder

    g = _tree(golden, "hf_encoder/")
    cfg = encoder.Encoder.default_config().set(
        name="enc", vocab_size=24, dim=12, pad_token_id=0,
        emb=encoder.bert_embedding_config(max_position_embeddings=11, layer_norm_epsilon=1e-12, type_vocab_size=1),
        transformer=encoder.bert_transformer_config(num_layers=2, num_heads=4, layer_norm_epsilon=1e-12))
    layer = cfg.instantiate(parent=None)
    ids = g["inputs"]["input_ids"].long()
    out, _ = functional(layer, prng.PRNGKey(1), g["params"]["encoder"], dict(input_ids=ids, token_type_ids=torch.zeros_like(ids)),
                        is_training=False)
    live = (ids != 0)[..., None]
    torch.testing.assert_close(out * live, g["outputs"]["last_hidden_state"] * live, rtol=2e-4, atol=2e-5)


def test_t5_encoder(golden):
    """The T5 v1.1 encoder with the reference's parameter tree reproduces the hidden states the
    reference recorded from Hugging Face's ``T5EncoderModel``."""
    from axlearn_b200.common.t5 import t5_encoder_config
    from axlearn_b200.common.utils import flatten_items

    g = _tree(golden, "t5_encoder/")
    cfg = t5_encoder_config(vocab_size=128, dim=12, num_layers=2, num_attention_heads=3).set(name="t5")
    layer = cfg.instantiate(parent=None)
    init = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert {p: tuple(t.shape) for p, t in flatten_items(init)} == {p: tuple(t.shape) for p, t in flatten_items(g["params"])}
    ids = g["inputs"]["input_ids"].long()
    out, _ = functional(layer, prng.PRNGKey(1), g["params"], dict(input_ids=ids), is_training=False)
    live = (ids != 0)[..., None]
    torch.testing.assert_close(out * live, g["outputs"]["last_hidden_state"] * live, rtol=1e-4, atol=5e-6)


def test_llama_rope_attention(golden):
    """Multi-head attention with RoPE on q / k against outputs the reference recorded from the
    original Llama attention (weights given as ``[out, in]`` matrices)."""
    from axlearn_b200.common.attention import MultiheadAttention, RoFormerQKVLinear

    g = _tree(golden, "llama_attention/")
    dim, heads = 32, 4
    cfg = MultiheadAttention.default_config().set(
        name="rope", query_dim=dim, key_dim=dim, value_dim=dim, num_heads=heads,
        input_linear=RoFormerQKVLinear.default_config().set(rotary_value=False))
    layer = cfg.instantiate(parent=None)
    state = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    for name, key in (("q_proj", "wq"), ("k_proj", "wk"), ("v_proj", "wv")):
        state["i_proj"]["i_proj"][name]["weight"] = g["params"][key].t().reshape(dim, heads, dim // heads).contiguous()
        if "bias" in state["i_proj"]["i_proj"][name]:
            state["i_proj"]["i_proj"][name]["bias"].zero_()
    state["o_proj"]["weight"] = g["params"]["wo"].reshape(dim, heads, dim // heads).contiguous()
    if "bias" in state["o_proj"]:
        state["o_proj"]["bias"].zero_()
    out, _ = functional(layer, prng.PRNGKey(0), state, dict(query=g["inputs"]["x"]), is_training=False)
    torch.testing.assert_close(out.data, g["outputs"]["data"].reshape(4, 100, -1), rtol=1e-4, atol=1e-5)


def test_llama_rope_frequencies(golden):
    from axlearn_b200.common.attention import RoFormerSinusoidalPositionalEmbedding

    g = _tree(golden, "llama_freqs_1e6/")
    dim, max_len, theta = int(g["params"]["dim"]), int(g["params"]["max_len"]), float(g["params"]["theta"])
    layer = RoFormerSinusoidalPositionalEmbedding.default_config().set(name="rope", dim=dim, theta=theta).instantiate(parent=None)
    table, _ = functional(layer, None, {}, dict(positions=torch.arange(max_len)[None]), is_training=False)
    sin, cos = table[0].chunk(2, dim=-1)
    torch.testing.assert_close(cos, g["outputs"]["real"], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(sin, g["outputs"]["imag"], rtol=1e-4, atol=1e-5)


def test_roberta_attention_and_layer(golden):
    from axlearn_b200.common.attention import TransformerAttentionLayer, TransformerLayer, scaled_hidden_dim

    g = _tree(golden, "roberta_attention/")
    cfg = TransformerAttentionLayer.default_config().set(name="att", target_dim=16, source_dim=16, structure="postnorm")
    cfg.attention.set(num_heads=4)
    layer = cfg.instantiate(parent=None)
    out, _ = functional(layer, prng.PRNGKey(0), g["params"], dict(target=g["inputs"]["target"]), is_training=True)
    torch.testing.assert_close(out.data, g["outputs"]["data"], rtol=1e-4, atol=1e-5)

    g = _tree(golden, "roberta_layer/")
    cfg = TransformerLayer.default_config().set(name="layer", input_dim=16)
    cfg.self_attention.set(structure="postnorm")
    cfg.feed_forward.set(structure="postnorm", activation="nn.silu", hidden_dim=scaled_hidden_dim(4))
    cfg.feed_forward.linear1.set(bias=True)
    cfg.feed_forward.linear2.set(bias=True)
    cfg.self_attention.attention.set(num_heads=4)
    layer = cfg.instantiate(parent=None)
    out, _ = functional(layer, prng.PRNGKey(0), g["params"], dict(data=g["inputs"]["data"]), is_training=True)
    torch.testing.assert_close(out.data, g["outputs"]["data"], rtol=1e-4, atol=1e-5)


def test_multihead_attention_xl(golden):
    """Transformer-XL relative attention inside a post-norm attention layer against the
    reference's recorded outputs (XLNet convention, scale on the logits)."""
    from axlearn_b200.common.attention import TransformerAttentionLayer
    from axlearn_b200.common.attention_xl import MultiheadAttentionXL, rel_pos_to_abs_pos

    x = torch.tensor([[0, 0, 1, 2, 3], [0, 4, 5, 6, 0], [7, 8, 9, 0, 0]])           # the docstring's example, t = 3
    assert rel_pos_to_abs_pos(x).tolist() == [[1, 2, 3], [4, 5, 6], [7, 8, 9]]
    g = _tree(golden, "attention_xl/")
    cfg = TransformerAttentionLayer.default_config().set(
        name="xl", target_dim=6, source_dim=6, structure="postnorm",
        attention=MultiheadAttentionXL.default_config().set(num_heads=2))
    cfg.attention.output_linear.bias = False
    layer = cfg.instantiate(parent=None)
    from axlearn_b200.common.utils import flatten_items

    init = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert {p: tuple(t.shape) for p, t in flatten_items(init)} == {p: tuple(t.shape) for p, t in flatten_items(g["params"])}
    out, _ = functional(layer, prng.PRNGKey(0), g["params"],
                        dict(target=g["inputs"]["target"], attention_logit_biases=g["inputs"]["attention_logit_biases"]),
                        is_training=True)
    torch.testing.assert_close(out.data, g["outputs"]["data"], rtol=1e-4, atol=6e-6)


def test_losses(golden):
    from axlearn_b200.common import loss

    g = _tree(golden, "loss_negative_cosine_similarity_loss_against_torch/")
    got, aux = loss.negative_cosine_similarity_loss(
        g["inputs"]["predictions"], g["inputs"]["targets"], live_targets=g["inputs"]["live_targets"])
    torch.testing.assert_close(got.double(), g["outputs"]["ref_loss"].double(), rtol=1e-5, atol=1e-6)
    assert aux["cosine_similarity"].shape == (2, 4)
    g = _tree(golden, "loss_koleo_loss_wo_norm/")
    torch.testing.assert_close(loss.koleo_loss(g["inputs"]["embeddings"], eps=1e-8).double(),
                               g["outputs"]["ref_loss"].double(), rtol=1e-5, atol=1e-6)
    g = _tree(golden, "loss_koleo_loss_w_norm/")
    torch.testing.assert_close(loss.koleo_loss(g["inputs"]["embeddings"], eps=1e-8, normalize_embedding=False).double(),
                               g["outputs"]["ref_loss"].double(), rtol=1e-5, atol=1e-6)
    logits, targets = torch.tensor([[2.0, 1.0, 0.0]]), torch.tensor([[0.0, 1.0, 0.0]])
    assert loss.categorical_hinge_loss(logits, targets).item() == 2.0
    torch.testing.assert_close(loss.sigmoid_cross_entropy_with_logits(torch.tensor([0.0]), torch.tensor([1.0])),
                               torch.tensor([0.6931472]))
    a, b = torch.randn(2, 4, 4, 3), torch.randn(2, 4, 4, 3)
    torch.testing.assert_close(loss.bilinear_mean_squared_error(a, b, shape=(2, 4, 4, 3)), (a - b).square().mean())
    assert loss.bilinear_mean_squared_error(a, b, shape=(2, 2, 2, 3)).item() < (a - b).square().mean().item()


def test_giou_and_degenerate_koleo(golden):
    from axlearn_b200.common import loss

    g = _tree(golden, "loss_giou_loss/")
    got = loss.giou_loss(predictions=g["inputs"]["predictions"], targets=g["inputs"]["targets"])
    got = got[0] if isinstance(got, tuple) else got
    torch.testing.assert_close(got.double().reshape(-1).mean(), g["outputs"]["ref_loss"].double().reshape(-1).mean(),
                               rtol=1e-4, atol=1e-5)
    g = _tree(golden, "loss_koleo_loss_zero_dist/")
    torch.testing.assert_close(loss.koleo_loss(g["inputs"]["embeddings"], eps=1e-8).double(),
                               g["outputs"]["ref_loss"].double(), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("mode", ["max", "sum"])
def test_splade_pooling(golden, mode):
    from axlearn_b200.common.layers import Linear
    from axlearn_b200.common.splade import SpladePooling

    cfg = SpladePooling.default_config().set(name="splade", input_dim=32, output_dim=64, splade_mode=mode)
    cfg.vocab_mapping.inner_head = Linear.default_config().set(bias=False)
    layer = cfg.instantiate(parent=None)
    for case in ("no_padding", "with_padding"):
        g = _tree(golden, f"splade_test_splade_pooling_{mode}_{case}/")
        paddings = None if case == "no_padding" else 1.0 - g["inputs"]["paddings"]      # stored as a validity mask
        got, _ = functional(layer, None, g["params"], dict(tokens=g["inputs"]["tokens"], paddings=paddings),
                            is_training=True)
        torch.testing.assert_close(got, g["outputs"]["values"], rtol=1e-5, atol=1e-5)


def test_distilbert(golden):
    from axlearn_b200.common.distilbert import set_distilbert_config
    from axlearn_b200.common.text_encoder import TEXT_EMBEDDINGS

    g = _tree(golden, "distilbert_test_distilbert/")
    vocab = g["params"]["encoder"]["emb"]["token_emb"]["weight"].shape[0]   # only the rows the inputs use are stored
    cfg = set_distilbert_config(pad_token_id=0, max_seq_len=12, vocab_size=vocab, num_layers=1, model_dim=32,
                                num_heads=8, feed_forward_dim=64, feed_forward_act="exact_gelu", dropout_rate=0)
    layer = cfg.set(name="test").instantiate(parent=None)
    got, _ = functional(layer, None, g["params"], dict(input_ids=g["inputs"]["input_ids"]), is_training=False)
    torch.testing.assert_close(got[TEXT_EMBEDDINGS], g["outputs"]["text_embeddings"], rtol=1e-5, atol=1e-5)


def test_bert_text_embedding_stream_encoder(golden):
    from axlearn_b200.common.text_dual_encoder import POSITIVE_EMBEDDINGS, POSITIVE_INPUT_IDS
    from axlearn_b200.common.utils_text_dual_encoder import bert_text_embedding_stream_encoder_config

    g = _tree(golden, "tde_test_bert_stream_encoder_config/")
    vocab = g["params"]["encoder"]["emb"]["token_emb"]["weight"].shape[0]   # only the rows the inputs use are stored
    cfg = bert_text_embedding_stream_encoder_config(
        pad_token_id=0, max_seq_len=12, vocab_size=vocab, num_layers=3, hidden_dim=32, output_dim=32, num_heads=8,
        output_proj=None, output_norm=None, remat=False)
    layer = cfg.set(name="test").instantiate(parent=None)
    batch = {POSITIVE_INPUT_IDS: g["inputs"]["input_ids"][:, None]}
    got, _ = functional(layer, None, dict(text_encoder=g["params"]), dict(input_batch=batch), is_training=False)
    torch.testing.assert_close(got[POSITIVE_EMBEDDINGS], g["outputs"]["emb"][:, None], rtol=1e-5, atol=1e-5)
