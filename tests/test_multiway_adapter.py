"""Multiway transformer routing; wrapping a torch.nn.Module as a layer."""
import torch

from axlearn_b200.common import multiway_transformer as mw
from axlearn_b200.common import prng
from axlearn_b200.common.adapter_torch import config_for_torch_module
from axlearn_b200.common.module import functional
from axlearn_b200.common.utils import flatten_items, tree_map


def _encoder(num_ffn):
    cfg = mw.MultiModalEncoder.default_config().set(name="enc", output_dim=16, vocab_size=30, num_layers=2,
                                                    image_size=(16, 16), patch_size=(8, 8), max_text_len=5)
    cfg.layer.num_ffn = num_ffn
    cfg.layer.self_attention.attention.num_heads = 2
    return cfg.instantiate(parent=None)


def test_each_modality_uses_its_own_expert():
    enc = _encoder(2)
    params = enc.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    ids = torch.tensor([[3, 4, 5, 0, 0], [6, 7, 8, 9, 2]])
    image = torch.randn(2, 16, 16, 3)
    inputs = {mw.TEXT_MODALITY: ids, mw.IMAGE_MODALITY: image, mw.TEXT_IMAGE_MODALITY: {0: ids, 1: image}}
    out, _ = functional(enc, None, params, [inputs], is_training=False)
    assert {k: v.shape for k, v in out.items()} == {0: (2, 1, 16), 1: (2, 1, 16), 2: (2, 1, 16)}
    # Perturbing the image expert changes image and fused outputs, not text.
    changed = tree_map(lambda t: t.clone(), params)
    for i in range(2):
        changed[f"layer{i}"]["feed_forward1"]["linear2"]["weight"] *= -2.0
    out2, _ = functional(enc, None, changed, [inputs], is_training=False)
    torch.testing.assert_close(out2[0], out[0])
    assert not torch.allclose(out2[1], out[1]) and not torch.allclose(out2[2], out[2])
    # With a fused expert the fused sequence no longer touches the single-modality experts.
    fused = _encoder(3)
    p3 = fused.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    a, _ = functional(fused, None, p3, [{2: {0: ids, 1: image}}], is_training=False)
    c3 = tree_map(lambda t: t.clone(), p3)
    for i in range(2):
        c3[f"layer{i}"]["feed_forward1"]["linear2"]["weight"] *= -2.0
    b, _ = functional(fused, None, c3, [{2: {0: ids, 1: image}}], is_training=False)
    torch.testing.assert_close(a[2], b[2])


def test_torch_module_as_a_layer():
    def make(width=8):
        return torch.nn.Sequential(torch.nn.Linear(4, width), torch.nn.BatchNorm1d(width), torch.nn.ReLU(),
                                   torch.nn.Linear(width, 2))

    layer = config_for_torch_module(make, width=6).set(name="wrapped").instantiate(parent=None)
    specs = dict(flatten_items(layer.create_parameter_specs_recursively(), is_leaf=lambda s: hasattr(s, "mesh_axes")))
    assert specs["0/weight"].shape == (6, 4) and specs["1/running_mean"].shape == (6,) and "3/bias" in specs
    p1 = layer.initialize_parameters_recursively(prng.PRNGKey(0))
    p2 = layer.initialize_parameters_recursively(prng.PRNGKey(0))
    p3 = layer.initialize_parameters_recursively(prng.PRNGKey(1))
    torch.testing.assert_close(p1["0"]["weight"], p2["0"]["weight"])
    assert not torch.allclose(p1["0"]["weight"], p3["0"]["weight"])
    x = torch.randn(5, 4)
    params = tree_map(lambda t: t.clone().requires_grad_(t.is_floating_point()), p1)
    y, _ = functional(layer, None, params, [x], is_training=False)
    ref = make(6)
    ref.load_state_dict({k.replace("/", "."): v for k, v in flatten_items(p1)})
    torch.testing.assert_close(y, ref.eval()(x))
    y.sum().backward()
    assert params["0"]["weight"].grad is not None and params["3"]["bias"].grad.abs().sum() > 0
    # The framework's parameters drive the computation, not the module's own copies.
    zeroed = tree_map(lambda t: torch.zeros_like(t), p1)
    zeroed["1"]["running_var"] = torch.ones(6)
    z, _ = functional(layer, None, zeroed, [x], is_training=False)
    assert z.abs().sum() == 0
