import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.vision import virtex
from axlearn_b200.vision.metrics_vqa import normalize_answer, vqa_accuracy, vqa_accuracy_batch
from axlearn_b200.vision.resnet import named_resnet_config


def test_reverse_within_length():
    ids = torch.tensor([[1, 5, 6, 2, 0, 0], [1, 7, 2, 0, 0, 0]])
    assert virtex.reverse_within_length(ids, 0).tolist() == [[2, 6, 5, 1, 0, 0], [2, 7, 1, 0, 0, 0]]


def test_virtex_bidirectional_loss_depends_on_the_image():
    dec = virtex.caption_decoder_config(vocab_size=20, dim=16, num_layers=1, num_heads=2, max_len=8)
    cfg = virtex.VirTexModel.default_config().set(
        name="virtex", visual=named_resnet_config("resnet18").set(hidden_dim=4, num_blocks_per_stage=(1, 1, 1, 1)),
        textual_dim=16, forward_decoder=dec, backward_decoder=dec.clone())
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert "backward_decoder" in params and "visual_projection" in params
    batch = dict(image=torch.randn(2, 64, 64, 3), caption_tokens=torch.tensor([[1, 5, 6, 7, 2, 0], [1, 9, 2, 0, 0, 0]]))
    (loss, aux), col = functional(model, prng.PRNGKey(1), params, [batch], is_training=False, drop_output_collections=())
    assert aux["visual_tokens"].shape == (2, 4, 16) and aux["forward_logits"].shape == (2, 5, 20)
    assert torch.isfinite(loss)
    (loss2, _), _ = functional(model, prng.PRNGKey(1), params, [dict(batch, image=batch["image"] * 3 + 1)], is_training=False)
    assert not torch.allclose(loss, loss2)
    uni = cfg.clone(bidirectional=False).instantiate(parent=None)
    p1 = {k: v for k, v in params.items() if k != "backward_decoder"}
    (loss_f, _), _ = functional(uni, prng.PRNGKey(1), p1, [batch], is_training=False)
    assert loss_f < loss


def test_vqa_accuracy():
    assert normalize_answer("The two Dogs.") == "2 dogs" and normalize_answer("dont know!") == "don't know"
    assert normalize_answer("1,000 people") == "1000 people"
    humans = ["2", "two", "2", "3", "2", "two dogs", "2", "4", "2", "2"]
    assert vqa_accuracy("Two", humans) == pytest.approx(1.0)           # 7 of 10 say 2
    assert vqa_accuracy("3", humans) == pytest.approx(0.3)             # one human: 1/3 on nine subsets, 0 on one
    assert vqa_accuracy("cat", humans) == 0.0
    out = vqa_accuracy_batch(["two", "cat"], [humans, humans])
    assert out["vqa_accuracy"] == pytest.approx(0.5) and out["num_examples"] == 2
