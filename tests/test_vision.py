"""Vision: ResNet, image classification, CLIP-style dual encoder, detection utilities."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.attention import StackedTransformerLayer
from axlearn_b200.common.encoder import VisionTransformer
from axlearn_b200.common.module import functional
from axlearn_b200.common.utils import flatten_items
from axlearn_b200.vision import detection_utils as det
from axlearn_b200.vision.clip import CLIPModel, StreamEncoder, symmetric_contrastive_loss_from_logits
from axlearn_b200.vision.image_classification import ImageClassificationModel
from axlearn_b200.vision.resnet import ResNet, ResidualBlock, named_resnet_config


def _init(layer):
    return layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")


def test_resnet_endpoints_and_param_counts():
    cfg = named_resnet_config("resnet18").set(name="r18")
    net = cfg.instantiate(parent=None)
    params = _init(net)
    n = sum(t.numel() for p, t in flatten_items(params) if "moving_" not in p)
    assert n == 11_176_512                      # torchvision resnet18 without its fc layer
    out, oc = functional(net, prng.PRNGKey(1), params, [torch.randn(2, 64, 64, 3)], is_training=True,
                         drop_output_collections=())
    assert {k: tuple(v.shape) for k, v in out.items()} == {
        "2": (2, 16, 16, 64), "3": (2, 8, 8, 128), "4": (2, 4, 4, 256), "5": (2, 2, 2, 512), "embedding": (2, 512)}
    assert "moving_mean" in oc.state_updates["stem"]["norm1"]
    r50 = named_resnet_config("resnet50").set(name="r50").instantiate(parent=None)
    specs = r50.create_parameter_specs_recursively()
    import math
    n50 = sum(math.prod(s.shape) for p, s in flatten_items(specs, is_leaf=lambda x: hasattr(x, "mesh_axes")) if "moving_" not in p)
    assert n50 == 23_508_032                    # torchvision resnet50 without its fc layer
    assert r50.endpoints_dims["embedding"] == 2048


def test_image_classification_overfits_two_images():
    backbone = ResNet.default_config().set(hidden_dim=8, num_blocks_per_stage=(1, 1))
    backbone.stage.block = ResidualBlock.default_config()
    model = ImageClassificationModel.default_config().set(name="clf", backbone=backbone, num_classes=3,
                                                          label_smoothing=0.0).instantiate(parent=None)
    params = _init(model)
    leaves = [t.requires_grad_() for p, t in flatten_items(params) if "moving_" not in p]
    opt = torch.optim.Adam(leaves, lr=1e-2)
    torch.manual_seed(0)
    batch = {"image": torch.randn(4, 32, 32, 3), "label": torch.tensor([0, 2, 1, -1])}
    first = None
    for step in range(40):
        (loss, out), oc = functional(model, prng.PRNGKey(step), params, dict(input_batch=batch), is_training=True)
        first = first if first is not None else loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < 0.2 * first
    assert float(oc.summaries["accuracy"].mean) == 1.0 and int(oc.summaries["accuracy"].weight) == 3


def _clip():
    vit = VisionTransformer.default_config().set(image_size=(16, 16), patch_size=(8, 8), dim=32, num_classes=2)
    vit.transformer.set(num_layers=1)
    vit.transformer.layer.self_attention.attention.num_heads = 4
    vit.transformer.layer.feed_forward.hidden_dim = 64
    from axlearn_b200.common.encoder import CausalEncoder

    text = CausalEncoder.default_config().set(dim=32, vocab_size=50, pad_token_id=0)
    text.transformer.set(num_layers=1)
    text.transformer.layer.self_attention.attention.num_heads = 4
    text.transformer.layer.feed_forward.hidden_dim = 64
    from axlearn_b200.common.embedding import LearnedPositionalEmbedding

    text.emb.pos_emb = LearnedPositionalEmbedding.default_config().set(shape=(8,))
    return CLIPModel.default_config().set(
        name="clip",
        image_stream=StreamEncoder.default_config().set(encoder=vit, encoder_dim=32, output_dim=16, input_key="image"),
        text_stream=StreamEncoder.default_config().set(encoder=text, encoder_dim=32, output_dim=16, input_key="text"))


def test_clip_contrastive_training_aligns_pairs():
    assert symmetric_contrastive_loss_from_logits(torch.eye(4) * 50).item() < 1e-6
    model = _clip().instantiate(parent=None)
    params = _init(model)
    leaves = [t.requires_grad_() for _, t in flatten_items(params)]
    opt = torch.optim.Adam(leaves, lr=3e-3)
    torch.manual_seed(0)
    batch = {"image": torch.randn(4, 16, 16, 3), "text": torch.randint(1, 50, (4, 6))}
    batch["text"][0, 4:] = 0
    losses = []
    for step in range(60):
        (loss, out), oc = functional(model, prng.PRNGKey(step), params, dict(input_batch=batch), is_training=True)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.3 * losses[0]
    assert out["image_embedding"].shape == (4, 16)
    torch.testing.assert_close(out["image_embedding"].norm(dim=-1), torch.ones(4))
    assert float(oc.summaries["i2t_accuracy"]) == 1.0


def test_box_utilities():
    a = torch.tensor([[0.0, 0.0, 10.0, 10.0], [5.0, 5.0, 15.0, 15.0]])
    b = torch.tensor([[0.0, 0.0, 10.0, 10.0], [20.0, 20.0, 30.0, 30.0]])
    iou = det.pairwise_iou(a, b)
    assert iou[0, 0] == 1.0 and iou[0, 1] == 0.0 and iou[1, 0].item() == pytest.approx(25 / 175)
    anchors = torch.tensor([[2.0, 2.0, 12.0, 14.0]])
    boxes = torch.tensor([[1.0, 3.0, 9.0, 20.0]])
    w = (10.0, 10.0, 5.0, 5.0)
    torch.testing.assert_close(det.decode_boxes(det.encode_boxes(boxes, anchors, w), anchors, w), boxes)
    assert det.clip_boxes(torch.tensor([[-5.0, 2.0, 50.0, 70.0]]), (40, 60)).tolist() == [[0.0, 2.0, 40.0, 60.0]]
    anc = det.generate_anchors(image_shape=(64, 64), min_level=3, max_level=4, num_scales=2, aspect_ratios=(1.0, 2.0))
    assert anc[3].shape == (8 * 8 * 4, 4) and anc[4].shape == (4 * 4 * 4, 4)
    first = anc[3][0]
    assert ((first[:2] + first[2:]) / 2).tolist() == [4.0, 4.0]
    assert det.box_area(anc[3][:1]).item() == pytest.approx((4.0 * 8) ** 2, rel=1e-5)
    # NMS keeps the best of each overlapping cluster, padded to the requested size.
    bx = torch.tensor([[0, 0, 10, 10], [1, 1, 11, 11], [20, 20, 30, 30], [0, 0, 9, 9]], dtype=torch.float32)
    idx, valid = det.non_max_suppression(bx, torch.tensor([0.9, 0.8, 0.7, 0.95]), iou_threshold=0.5, max_output_size=3)
    assert idx.tolist() == [3, 2, -1] and valid.tolist() == [True, True, False]


def test_roi_align_on_a_linear_ramp():
    """On f(y, x) = y + 10 x bilinear sampling is exact: every cell is the ramp at its centre."""
    ys, xs = torch.meshgrid(torch.arange(8.0), torch.arange(8.0), indexing="ij")
    feat = (ys + 0.5 + 10 * (xs + 0.5))[..., None]            # value at the pixel centre
    out = det.roi_align(feat, torch.tensor([[2.0, 2.0, 6.0, 6.0]]), output_size=2, sampling_ratio=2)
    want = torch.tensor([[3 + 30.0, 3 + 50.0], [5 + 30.0, 5 + 50.0]])
    torch.testing.assert_close(out[0, :, :, 0], want)


def test_retinanet_learns_to_find_a_square():
    from axlearn_b200.vision.retinanet import FPN, RetinaNetModel, label_anchors, sigmoid_focal_loss

    # Focal loss: gamma = 0 and alpha = 0.5 is half the plain cross entropy.
    logits, targets = torch.randn(5, 3), torch.randint(0, 2, (5, 3)).float()
    torch.testing.assert_close(
        sigmoid_focal_loss(logits, targets, alpha=0.5, gamma=0.0),
        0.5 * torch.nn.functional.binary_cross_entropy_with_logits(logits, targets, reduction="none"))
    anchors = torch.tensor([[0.0, 0, 10, 10], [0, 0, 7, 10], [30, 30, 40, 40]])
    cls, boxes, pos = label_anchors(anchors, torch.tensor([[0.0, 0, 10, 10], [0, 0, 0, 0]]), torch.tensor([2, -1]))
    assert cls.tolist() == [2, 2, -1] and pos.tolist() == [True, True, False]
    cls2, _, _ = label_anchors(anchors, torch.tensor([[0.0, 0, 10, 22]]), torch.tensor([1]))
    assert cls2.tolist() == [-2, -1, -1]                    # IoU 0.45: neither positive nor background

    backbone = ResNet.default_config().set(hidden_dim=8, num_blocks_per_stage=(1, 1, 1))
    backbone.stage.block = ResidualBlock.default_config()
    cfg = RetinaNetModel.default_config().set(
        name="retina", backbone=backbone, num_classes=2, num_scales=1, aspect_ratios=(1.0,), anchor_size=3.0,
        fpn=FPN.default_config().set(hidden_dim=16, min_level=3, max_level=4))
    cfg.head.num_layers = 1
    model = cfg.instantiate(parent=None)
    params = _init(model)
    torch.manual_seed(0)
    image = torch.zeros(2, 64, 64, 3)
    image[0, 16:40, 16:40] = 1.0
    image[1, 24:48, 8:32, 1] = 1.0
    batch = {"image": image,
             "groundtruth_boxes": torch.tensor([[[16.0, 16, 40, 40]], [[24.0, 8, 48, 32]]]),
             "groundtruth_classes": torch.tensor([[0], [1]])}
    out0, _ = functional(model, prng.PRNGKey(0), params, dict(input_batch=batch), is_training=False, method="predict")
    assert out0["class_outputs"].shape == (2, 8 * 8 + 4 * 4, 2) and out0["anchors"].shape == (80, 4)
    assert torch.sigmoid(out0["class_outputs"]).mean().item() == pytest.approx(0.01, abs=0.02)   # prior probability
    leaves = [t.requires_grad_() for p, t in flatten_items(params) if "moving_" not in p]
    opt = torch.optim.Adam(leaves, lr=3e-3)
    first = None
    for step in range(150):
        (loss, _), oc = functional(model, prng.PRNGKey(step), params, dict(input_batch=batch), is_training=True)
        first = first if first is not None else loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < 0.2 * first and float(oc.summaries["num_positive_anchors"]) >= 1
    with torch.no_grad():
        dets, _ = functional(model, prng.PRNGKey(0), params, dict(input_batch=batch, score_threshold=0.3),
                             is_training=True, method="detect")
    for i, want_cls in enumerate([0, 1]):
        assert len(dets[i]["scores"]) >= 1 and dets[i]["classes"][0].item() == want_cls
        iou = det.pairwise_iou(dets[i]["boxes"][:1], batch["groundtruth_boxes"][i])
        assert iou.item() > 0.5
