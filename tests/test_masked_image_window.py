"""Masked image modelling and windowed attention."""
import numpy as np
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.vision import masked_image_model as mim
from axlearn_b200.vision import window_attention as wa


def test_mask_generator_masks_the_requested_number_in_blocks():
    gen = mim.MaskingGenerator(input_size=(14, 14), num_masking_patches=75, min_mask_patches=16)
    masks = [gen(seed) for seed in range(8)]
    assert all(m.sum() == 75 and m.shape == (14, 14) for m in masks)
    assert not np.array_equal(masks[0], masks[1]) and np.array_equal(gen(3), gen(3))
    # Blocks: most masked cells have a masked 4-neighbour.
    m = masks[0]
    pad = np.pad(m, 1)
    neigh = pad[:-2, 1:-1] | pad[2:, 1:-1] | pad[1:-1, :-2] | pad[1:-1, 2:]
    assert (neigh & m).sum() / m.sum() > 0.8


def _model(tokenizer):
    enc = mim.MaskedImageEncoder.default_config().set(image_size=(32, 32), patch_size=(8, 8), dim=16)
    enc.transformer.num_layers = 1
    enc.transformer.layer.self_attention.attention.num_heads = 2
    enc.transformer.layer.feed_forward.hidden_dim = 32
    return mim.MaskedImageModel.default_config().set(name="mim", tokenizer=tokenizer, encoder=enc).instantiate(parent=None)


def test_masked_image_model_with_discrete_and_feature_targets():
    image = torch.randn(3, 32, 32, 3)
    for tok in (mim.DiscreteImageTokenizer.default_config().set(patch_size=(8, 8), hidden_dim=8, vocab_size=32),
                mim.PatchFeatureTokenizer.default_config().set(patch_size=(8, 8))):
        model = _model(tok)
        params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
        (loss, aux), _ = functional(model, prng.PRNGKey(1), params, [dict(image=image)], is_training=True)
        assert aux["is_masked"].shape == (3, 16) and (aux["is_masked"].sum(-1) == 6).all()
        assert torch.isfinite(loss)
        # Only masked positions count: changing the prediction targets elsewhere leaves the loss alone.
        fixed = dict(image=image, is_masked=aux["is_masked"])
        (l1, a1), _ = functional(model, prng.PRNGKey(1), params, [fixed], is_training=False)
        torch.testing.assert_close(l1, loss)
    assert aux["labels"].shape == (3, 16, 8 * 8 * 3)


def test_window_partition_round_trip_and_locality():
    x = torch.randn(2, 10, 7, 4)
    windows, padded = wa.window_partition(x, 4)
    assert windows.shape == (2 * 3 * 2, 4, 4, 4) and padded == (12, 8)
    torch.testing.assert_close(wa.window_unpartition(windows, 4, padded, (10, 7)), x)
    cfg = wa.ViTDetTransformer.default_config().set(name="v", input_dim=8, num_layers=2, window_size=4,
                                                    global_attention_indices=[])
    cfg.layer.self_attention.attention.num_heads = 2
    cfg.layer.feed_forward.hidden_dim = 16
    net = cfg.instantiate(parent=None)
    params = net.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    a = torch.randn(1, 8, 8, 8)
    b = a.clone()
    b[0, 6, 6, 0] += 5.0                                         # lives in the bottom-right window
    ya, _ = functional(net, None, params, [a], is_training=False)
    yb, _ = functional(net, None, params, [b], is_training=False)
    torch.testing.assert_close(ya[0, :4], yb[0, :4])             # other windows are untouched
    assert not torch.allclose(ya[0, 4:, 4:], yb[0, 4:, 4:])
    glob = cfg.clone(global_attention_indices=[1]).instantiate(parent=None)
    ga, _ = functional(glob, None, params, [a], is_training=False)
    gb, _ = functional(glob, None, params, [b], is_training=False)
    assert not torch.allclose(ga[0, :4, :4], gb[0, :4, :4])      # a global block mixes windows
    odd, _ = functional(net, None, params, [torch.randn(1, 6, 5, 8)], is_training=False)
    assert odd.shape == (1, 6, 5, 8) and torch.isfinite(odd).all()
