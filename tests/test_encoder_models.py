"""Encoder-side model families: they build, run, mask padding correctly and learn."""

import torch

from axlearn_b200.common import encoder, prng
from axlearn_b200.common.attention import StackedTransformerLayer, TransformerLayer
from axlearn_b200.common.embedding import LearnedPositionalEmbedding, TransformerTextEmbeddings
from axlearn_b200.common.module import functional


def _stack(dim, heads=2, layers=2):
    layer = TransformerLayer.default_config()
    layer.self_attention.attention.num_heads = heads
    layer.feed_forward.hidden_dim = 2 * dim
    return StackedTransformerLayer.default_config().set(num_layers=layers, layer=layer)


def _emb(max_len=32):
    return TransformerTextEmbeddings.default_config().set(
        pos_emb=LearnedPositionalEmbedding.default_config().set(shape=(max_len,)))


def _sgd_steps(model, params, batch, steps=25, lr=0.1):
    params = {k: v for k, v in params.items()}
    from axlearn_b200.common.utils import flatten_items, tree_map

    params = tree_map(lambda t: t.clone().requires_grad_(True), params)
    losses = []
    for _ in range(steps):
        (loss, _), _ = functional(model, prng.PRNGKey(0), params, dict(input_batch=batch), is_training=True)
        grads = torch.autograd.grad(loss, [t for _, t in flatten_items(params)], allow_unused=True)
        with torch.no_grad():
            for (_, t), g in zip(flatten_items(params), grads):
                if g is not None:
                    t -= lr * g
        losses.append(loss.item())
    return losses


def test_encoder_ignores_padding_tokens():
    cfg = encoder.Encoder.default_config().set(name="enc", vocab_size=50, dim=16, emb=_emb(), transformer=_stack(16))
    enc = cfg.instantiate(parent=None)
    params = enc.initialize_parameters_recursively(prng.PRNGKey(0))
    ids = torch.tensor([[5, 6, 7, 0, 0], [5, 6, 7, 8, 9]])
    out, _ = functional(enc, None, params, [ids], is_training=False)
    ids2 = ids.clone()
    out2, _ = functional(enc, None, params, [torch.tensor([[5, 6, 7, 0, 0], [5, 6, 7, 11, 12]])], is_training=False)
    assert out.shape == (2, 5, 16)
    assert torch.allclose(out[0, :3], out2[0, :3], atol=1e-6)
    # Row 0's live positions do not depend on what sits in padding positions of the batch.
    short, _ = functional(enc, None, params, [ids[:1, :3]], is_training=False)
    assert torch.allclose(short[0], out[0, :3], atol=1e-5)
    del ids2


def test_causal_encoder_has_no_lookahead():
    cfg = encoder.CausalEncoder.default_config().set(name="enc", vocab_size=50, dim=16, emb=_emb(), transformer=_stack(16))
    enc = cfg.instantiate(parent=None)
    params = enc.initialize_parameters_recursively(prng.PRNGKey(0))
    a, _ = functional(enc, None, params, [torch.tensor([[5, 6, 7, 8]])], is_training=False)
    b, _ = functional(enc, None, params, [torch.tensor([[5, 6, 9, 10]])], is_training=False)
    assert torch.allclose(a[0, :2], b[0, :2], atol=1e-6) and not torch.allclose(a[0, 2], b[0, 2])


def test_bert_mlm_learns():
    cfg = encoder.BertModel.default_config().set(name="bert", vocab_size=40, dim=16)
    cfg.encoder.set(emb=_emb(), transformer=_stack(16))
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0))
    assert set(params["head"]) == {"transform", "output_bias"} and set(params["head"]["transform"]) == {"linear", "norm"}
    ids = torch.randint(4, 40, (4, 8))
    labels = torch.zeros_like(ids)
    labels[:, 2] = ids[:, 2]
    masked = ids.clone()
    masked[:, 2] = 3
    batch = {"input_ids": masked, "target_labels": labels}
    losses = _sgd_steps(model, params, batch)
    assert losses[-1] < 0.6 * losses[0]
    out, _ = functional(model, None, params, dict(input_batch=batch), is_training=False, method="predict")
    assert out["logits"].shape == (4, 8, 40) and out["sequence_output"].shape == (4, 8, 16)


def test_bert_sequence_classification_learns():
    cfg = encoder.BertModel.default_config().set(
        name="bert", vocab_size=40, dim=16, head=encoder.BertSequenceClassificationHead.default_config().set(num_classes=3))
    cfg.encoder.set(emb=_emb(), transformer=_stack(16))
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0))
    assert set(params["head"]) == {"pooler", "output"}
    batch = {"input_ids": torch.randint(4, 40, (4, 8)), "target_labels": torch.tensor([0, 1, 2, 1])}
    losses = _sgd_steps(model, params, batch)
    assert losses[-1] < 0.6 * losses[0]
    out, _ = functional(model, None, params, dict(input_batch=batch), is_training=False, method="predict")
    assert out["logits"].shape == (4, 3) and out["pooled_output"].shape == (4, 16)


def test_encoder_decoder_learns_to_copy():
    cfg = encoder.encoder_decoder_config(vocab_size=30, dim=16, num_layers=1, num_heads=2, max_len=16).set(name="s2s")
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0))
    src = torch.randint(3, 30, (4, 6))
    tgt_in = torch.cat([torch.ones(4, 1, dtype=torch.long), src[:, :-1]], dim=1)
    batch = {"source": {"input_ids": src}, "target": {"input_ids": tgt_in}, "target_labels": src}
    losses = _sgd_steps(model, params, batch, steps=40, lr=0.2)
    assert losses[-1] < 0.7 * losses[0]


def test_vision_transformer_shapes_and_learning():
    cfg = encoder.VisionTransformer.default_config().set(
        name="vit", image_size=(16, 16), patch_size=(4, 4), dim=16, num_classes=5, transformer=_stack(16, layers=1))
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0))
    batch = {"image": torch.randn(6, 16, 16, 3), "label": torch.tensor([0, 1, 2, 3, 4, 0])}
    out, _ = functional(model, None, params, dict(input_batch=batch), is_training=False, method="predict")
    assert out["encoded"].shape == (6, 17, 16) and out["logits"].shape == (6, 5)
    losses = _sgd_steps(model, params, batch, steps=30, lr=0.1)
    assert losses[-1] < 0.7 * losses[0]
