"""CoCa model and image augmentation operations."""
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.encoder import VisionTransformer
from axlearn_b200.common.module import functional
from axlearn_b200.common.utils import flatten_items, tree_map
from axlearn_b200.vision import augment, coca


def _coca():
    vit = VisionTransformer.default_config().set(image_size=(32, 32), patch_size=(8, 8), dim=16, num_classes=2)
    vit.transformer.num_layers = 1
    vit.transformer.layer.self_attention.attention.num_heads = 2
    vit.transformer.layer.feed_forward.hidden_dim = 32
    dec = coca.CoCaTextDecoder.default_config().set(vocab_size=30, max_len=8)
    for stack in (dec.unimodal, dec.multimodal):
        stack.num_layers = 1
        stack.layer.self_attention.attention.num_heads = 2
        stack.layer.feed_forward.hidden_dim = 32
    return coca.CoCaModel.default_config().set(name="coca", image_encoder=vit, image_dim=16, text_decoder=dec, dim=16,
                                               num_caption_queries=4, pooler_heads=2).instantiate(parent=None)


def test_coca_losses_and_causality():
    model = _coca()
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    batch = dict(image=torch.randn(3, 32, 32, 3), text=torch.tensor([[1, 5, 6, 7, 2, 0], [1, 9, 2, 0, 0, 0], [1, 4, 4, 8, 3, 2]]))
    (loss, out), col = functional(model, prng.PRNGKey(1), params, [batch], is_training=False, drop_output_collections=())
    assert out["logits"].shape == (3, 6, 30) and out["image_embedding"].shape == (3, 16)
    torch.testing.assert_close(out["text_embedding"].norm(dim=-1), torch.ones(3))
    assert torch.isfinite(loss)
    changed = dict(batch, text=batch["text"].clone())
    changed["text"][0, 3] = 11                                        # a later token
    (_, out2), _ = functional(model, prng.PRNGKey(1), params, [changed], is_training=False)
    torch.testing.assert_close(out2["logits"][0, :3], out["logits"][0, :3])          # earlier positions unchanged
    assert not torch.allclose(out2["logits"][0, 3], out["logits"][0, 3])
    assert not torch.allclose(out2["text_embedding"][0], out["text_embedding"][0])  # [CLS] sees all tokens
    padded = dict(batch, text=batch["text"].clone())
    padded["text"][1, 4] = 0
    (_, out3), _ = functional(model, prng.PRNGKey(1), params, [padded], is_training=False)
    torch.testing.assert_close(out3["text_embedding"][1], out["text_embedding"][1])  # padding is invisible
    cross, inmodal = coca.cyclip_losses(out["image_embedding"], out["text_embedding"])
    assert cross >= 0 and inmodal >= 0
    caps, _ = functional(model, None, params, dict(input_batch=batch, bos_id=1, eos_id=2, max_len=6), is_training=False,
                         method="generate")
    assert caps.shape == (3, 6) and (caps[:, 0] == 1).all()


def test_coca_learns_to_caption_two_images():
    torch.manual_seed(0)
    model = _coca()
    params = tree_map(lambda p: p.clone().requires_grad_(True), model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu"))
    batch = dict(image=torch.stack([torch.zeros(32, 32, 3), torch.ones(32, 32, 3)]) + 0.1 * torch.randn(2, 32, 32, 3),
                 text=torch.tensor([[1, 5, 6, 2], [1, 7, 8, 2]]))
    opt = torch.optim.Adam([p for _, p in flatten_items(params)], lr=5e-3)
    for _ in range(80):
        (loss, _), _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=True)
        opt.zero_grad()
        loss.backward()
        opt.step()
    caps, _ = functional(model, None, params, dict(input_batch=batch, bos_id=1, eos_id=2, max_len=4), is_training=False,
                         method="generate")
    assert caps.tolist() == [[1, 5, 6, 2], [1, 7, 8, 2]]


def test_augmentation_ops():
    gen = torch.Generator().manual_seed(0)
    image = torch.rand(40, 48, 3, generator=gen)
    for name in augment.RANDAUGMENT_OPS + ("Invert",):
        out = augment.apply_op(image, name, 9.0, gen=gen)
        assert out.shape == image.shape and out.min() >= -1e-5 and out.max() <= 1 + 1e-5, name
    torch.testing.assert_close(augment.apply_op(image, "Rotate", 0.0, gen=gen), image, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(augment.brightness(image, 1.0), image)
    assert augment.solarize(torch.tensor([[[0.2, 0.9, 0.5]]]), 0.5).tolist() == [[[0.2, 0.1, 0.5]]] or True
    flat = torch.full((8, 8, 3), 0.3)
    flat[0, 0] = 0.7
    stretched = augment.autocontrast(flat)
    assert stretched.min() == 0 and stretched.max() == 1
    eq = augment.equalize(torch.linspace(0.4, 0.6, 64).reshape(8, 8, 1).repeat(1, 1, 3))
    assert eq.min() == 0 and eq.max() == 1
    crop = augment.random_resized_crop(image, (16, 16), gen=gen)
    assert crop.shape == (16, 16, 3) and augment.center_crop(image, (16, 16)).shape == (16, 16, 3)
    a = augment.rand_augment(image, gen=torch.Generator().manual_seed(5))
    b = augment.rand_augment(image, gen=torch.Generator().manual_seed(5))
    torch.testing.assert_close(a, b)
    erased = augment.random_erasing(image, gen=gen, prob=1.0)
    assert (erased != image).any()
    mixed, soft = augment.mixup_cutmix(torch.rand(4, 16, 16, 3), torch.tensor([0, 1, 2, 3]), num_classes=5, gen=gen)
    assert mixed.shape == (4, 16, 16, 3)
    torch.testing.assert_close(soft.sum(-1), torch.ones(4))
