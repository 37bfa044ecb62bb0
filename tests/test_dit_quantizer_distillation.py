"""DiT blocks, vector quantisers and the distillation wrapper."""

import math

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.distillation import DistillationModel, soft_target_kl
from axlearn_b200.common.dit import DiT, DiTBlock, LabelEmbedding, TimeStepEmbedding
from axlearn_b200.common.module import functional
from axlearn_b200.common.quantizer import (
    KmeansVectorQuantizer,
    RandomVectorQuantizer,
    compute_code_coverage,
    compute_code_histogram,
    compute_code_pplx,
    quantize_by_nearest_neighbor,
)
from axlearn_b200.common.utils import flatten_items
from axlearn_b200.vision.image_classification import ImageClassificationModel
from axlearn_b200.vision.resnet import ResNet, ResidualBlock


def _init(layer):
    return layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")


def test_dit_block_is_identity_at_init_and_model_shapes():
    block = DiTBlock.default_config().set(name="b", input_dim=32, num_heads=4).instantiate(parent=None)
    params = _init(block)
    x, cond = torch.randn(2, 6, 32), torch.randn(2, 32)
    y, _ = functional(block, prng.PRNGKey(1), params, dict(inputs=x, condition=cond), is_training=False)
    torch.testing.assert_close(y, x)                     # adaLN-zero: all gates start at 0
    # Once the modulation is non-zero the condition matters.
    params["adaln"]["linear"]["weight"] = torch.randn_like(params["adaln"]["linear"]["weight"]) * 0.1
    y1, _ = functional(block, prng.PRNGKey(1), params, dict(inputs=x, condition=cond), is_training=False)
    y2, _ = functional(block, prng.PRNGKey(1), params, dict(inputs=x, condition=cond + 1), is_training=False)
    assert not torch.allclose(y1, x) and not torch.allclose(y1, y2)
    model = DiT.default_config().set(name="dit", image_size=(8, 8), patch_size=2, input_channels=4, output_channels=8,
                                     dim=32, num_layers=2, num_heads=4, num_classes=10).instantiate(parent=None)
    p = _init(model)
    img = torch.randn(3, 8, 8, 4)
    out, _ = functional(model, prng.PRNGKey(1), p, dict(image=img, timesteps=torch.tensor([0.0, 10.0, 999.0]),
                                                        labels=torch.tensor([1, 2, 3])), is_training=True)
    assert out.shape == (3, 8, 8, 8) and out.abs().sum() == 0          # zero-initialised final layer
    t_emb = TimeStepEmbedding.default_config().set(name="t", output_dim=16).instantiate(parent=None)
    e, _ = functional(t_emb, prng.PRNGKey(1), _init(t_emb), dict(positions=torch.tensor([0.0, 500.0])), is_training=False)
    assert e.shape == (2, 16) and not torch.allclose(e[0], e[1])
    lab = LabelEmbedding.default_config().set(name="l", num_classes=5, output_dim=8, dropout_rate=1.0).instantiate(parent=None)
    lp = _init(lab)
    dropped, _ = functional(lab, prng.PRNGKey(1), lp, dict(labels=torch.tensor([0, 3])), is_training=True)
    torch.testing.assert_close(dropped[0], lp["emb"]["weight"][5])     # everything maps to the null class
    kept, _ = functional(lab, prng.PRNGKey(1), lp, dict(labels=torch.tensor([0, 3])), is_training=False)
    torch.testing.assert_close(kept[1], lp["emb"]["weight"][3])


def test_nearest_neighbor_and_code_metrics():
    codebook = torch.tensor([[[0.0, 0.0]], [[1.0, 1.0]], [[5.0, 5.0]]])              # V=3, G=1, H=2
    x = torch.tensor([[[[0.2, -0.1]], [[4.0, 4.5]], [[0.9, 1.2]]]])
    ids, vec = quantize_by_nearest_neighbor(x, codebook=codebook)
    assert ids.reshape(-1).tolist() == [0, 2, 1]
    torch.testing.assert_close(vec[0, 1, 0], torch.tensor([5.0, 5.0]))
    hist = compute_code_histogram(torch.tensor([[[0], [0], [1], [2]]]), vocab_size=4, paddings=torch.tensor([[0, 0, 0, 1.0]]))
    assert hist.tolist() == [[2.0, 1.0, 0.0, 0.0]]
    assert compute_code_coverage(hist).item() == 0.5
    p = torch.tensor([2 / 3, 1 / 3])
    assert compute_code_pplx(hist).item() == pytest.approx(math.exp(-(p * p.log()).sum().item()), abs=1e-5)


def test_kmeans_quantizer_losses_and_straight_through():
    q = KmeansVectorQuantizer.default_config().set(name="q", codebook_dim=4, codebook_size=8, num_codebooks=2,
                                                   beta=0.25).instantiate(parent=None)
    params = _init(q)
    params["codebook"].requires_grad_()
    x = torch.randn(2, 5, 8, requires_grad=True)
    paddings = torch.zeros(2, 5)
    paddings[1, 3:] = 1
    out, oc = functional(q, prng.PRNGKey(1), params, dict(inputs=x, paddings=paddings), is_training=True)
    assert out.ids.shape == (2, 5, 2) and (out.ids[1, 3:] == -1).all() and (out.ids[0] >= 0).all()
    assert out.quantized_vectors.shape == (2, 5, 2, 4) and out.quantized_vectors[1, 3:].abs().sum() == 0
    # Forward value = codebook entries; gradient wrt the input = identity on live positions.
    g = torch.arange(2)
    torch.testing.assert_close(out.quantized_vectors[0, 0], params["codebook"][out.ids[0, 0], g].detach())
    out.quantized_vectors.sum().backward(retain_graph=True)
    assert torch.equal(x.grad[0], torch.ones(5, 8)) and x.grad[1, 3:].abs().sum() == 0
    x.grad = None
    out.loss.backward()
    assert params["codebook"].grad.abs().sum() > 0 and x.grad.abs().sum() > 0
    assert 0 < float(oc.summaries["codebook/coverage"].mean) <= 1


def test_random_quantizer_is_deterministic_and_untrained():
    q = RandomVectorQuantizer.default_config().set(name="rq", input_dim=16, codebook_dim=4, codebook_size=32,
                                                   num_codebooks=1).instantiate(parent=None)
    params = _init(q)
    x = torch.randn(2, 7, 16, requires_grad=True)
    out1, _ = functional(q, prng.PRNGKey(1), params, dict(inputs=x, paddings=torch.zeros(2, 7)), is_training=True)
    out2, _ = functional(q, prng.PRNGKey(2), params, dict(inputs=x, paddings=torch.zeros(2, 7)), is_training=True)
    assert torch.equal(out1.ids, out2.ids) and not out1.quantized_vectors.requires_grad
    torch.testing.assert_close(out1.quantized_vectors.norm(dim=-1), torch.ones(2, 7, 1))


def _clf(name):
    backbone = ResNet.default_config().set(hidden_dim=4, num_blocks_per_stage=(1,))
    backbone.stage.block = ResidualBlock.default_config()
    return ImageClassificationModel.default_config().set(name=name, backbone=backbone, num_classes=3)


def test_distillation_freezes_teacher_and_vanishes_for_equal_models():
    logits = torch.randn(4, 5)
    assert soft_target_kl(student_logits=logits, teacher_logits=logits, temperature=2.0).item() == pytest.approx(0, abs=1e-6)
    assert soft_target_kl(student_logits=logits, teacher_logits=logits + torch.randn(4, 5)).item() > 0
    model = DistillationModel.default_config().set(name="distill", teacher=_clf("teacher"), student=_clf("student"),
                                                   temperature=2.0, soft_target_weight=1.0).instantiate(parent=None)
    params = _init(model)
    leaves = dict(flatten_items(params))
    for t in leaves.values():
        t.requires_grad_()
    batch = {"image": torch.randn(4, 16, 16, 3), "label": torch.tensor([0, 1, 2, 1])}
    (loss, aux), _ = functional(model, prng.PRNGKey(1), params, dict(input_batch=batch), is_training=True)
    loss.backward()
    assert all(t.grad is None for p, t in leaves.items() if p.startswith("teacher/"))
    assert any(t.grad is not None and t.grad.abs().sum() > 0 for p, t in leaves.items() if p.startswith("student/"))
    # A student that equals the teacher has nothing to learn from it.
    same = {"teacher": params["teacher"], "student": params["teacher"]}
    (loss2, _), _ = functional(model, prng.PRNGKey(1), same, dict(input_batch=batch), is_training=False)
    assert loss2.item() == pytest.approx(0, abs=1e-6)
