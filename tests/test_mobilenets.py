"""MobileNetV3 / EfficientNet backbones: parameter counts against torchvision-known totals, shapes."""
import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.common.utils import flatten_items
from axlearn_b200.vision import mobilenets
from axlearn_b200.vision.image_classification import ImageClassificationModel


def _count(cfg, classes=1000):
    model = ImageClassificationModel.default_config().set(name="m", backbone=cfg, num_classes=classes).instantiate(parent=None)
    specs = model.create_parameter_specs_recursively()
    total = 0
    for path, spec in flatten_items(specs, is_leaf=lambda x: hasattr(x, "mesh_axes")):
        if "moving_" in path:
            continue
        n = 1
        for d in spec.shape:
            n *= d
        total += n
    return total


def test_parameter_counts_match_the_published_models():
    # torchvision: efficientnet_b0 5,288,548; mobilenet_v3_large 5,483,032; mobilenet_v3_small 2,542,856.
    assert _count(mobilenets.named_model_configs("efficientnet-b0")) == 5_288_548
    assert _count(mobilenets.named_model_configs("mobilenetv3-large-100")) == 5_483_032
    assert _count(mobilenets.named_model_configs("mobilenetv3-small-100")) == 2_542_856


def test_make_divisible():
    assert mobilenets.make_divisible(32 * 1.1) == 32 and mobilenets.make_divisible(40 * 1.2) == 48
    assert mobilenets.make_divisible(10, 8) == 16          # would lose more than 10 % otherwise
    assert mobilenets.round_features(16, 0.75) == 16


@pytest.mark.parametrize("name", ["mobilenetv3-small-minimal-075", "efficientnet-lite0", "efficientnetv2-s", "efficientnet-b2"])
def test_forward_endpoints(name):
    cfg = mobilenets.named_model_configs(name).set(name="net")
    net = cfg.instantiate(parent=None)
    params = net.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    out, _ = functional(net, prng.PRNGKey(1), params, [torch.randn(2, 64, 64, 3)], is_training=False)
    dims = net.endpoints_dims
    for level in ("1", "2", "3", "4", "5"):
        assert out[level].shape == (2, 64 // 2 ** int(level), 64 // 2 ** int(level), dims[level]), (name, level)
    assert out["embedding"].shape == (2, dims["embedding"])
    assert torch.isfinite(out["embedding"]).all()


def test_training_step_updates_batch_norm_state_and_uses_stochastic_depth():
    cfg = mobilenets.named_model_configs("mobilenetv3-small-100").set(name="net", peak_stochastic_depth_rate=0.2)
    net = cfg.instantiate(parent=None)
    params = net.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    out, col = functional(net, prng.PRNGKey(1), params, [torch.randn(4, 32, 32, 3)], is_training=True,
                          drop_output_collections=())
    updates = dict(flatten_items(col.state_updates))
    assert any(k.endswith("moving_mean") for k in updates)
    assert out["embedding"].shape == (4, 1024)
