"""Parameter noise: applied by the trainer, children before parents, gradients on clean parameters."""

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import GaussianParameterNoise
from axlearn_b200.common.layers import Linear
from axlearn_b200.common.module import functional
from tests.helpers import tiny_fuji_trainer_config


def test_noise_changes_what_the_layer_reads_but_not_the_parameters():
    cfg = Linear.default_config().set(name="lin", input_dim=8, output_dim=4, bias=False)
    clean = cfg.instantiate(parent=None)
    params = clean.initialize_parameters_recursively(prng.PRNGKey(0))
    assert not clean.has_parameter_noise()
    assert clean.apply_parameter_noise_recursively(prng.PRNGKey(1), params) is params
    noisy_cfg = cfg.clone(param_noise=GaussianParameterNoise.default_config().set(std=0.1, regex="weight"))
    noisy = noisy_cfg.instantiate(parent=None)
    assert noisy.has_parameter_noise()
    w = params["weight"].clone().requires_grad_()
    out = noisy.apply_parameter_noise_recursively(prng.PRNGKey(1), {"weight": w})
    assert out["weight"] is not w and not torch.equal(out["weight"], w)
    assert (out["weight"] - w).std().item() > 0.05
    again = noisy.apply_parameter_noise_recursively(prng.PRNGKey(1), {"weight": w})
    assert torch.equal(out["weight"], again["weight"])  # a function of the key
    x = torch.randn(3, 8)
    y, _ = functional(noisy, prng.PRNGKey(2), out, [x], is_training=True)
    y.sum().backward()
    assert w.grad is not None and torch.allclose(w.grad, x.sum(0)[:, None].expand(8, 4))


def test_trainer_applies_noise_each_step(tmp_path):
    def run(std):
        cfg = tiny_fuji_trainer_config(tmp_path / f"s{std}", max_step=3, layers=1, vocab=256, save_every_n_steps=100)
        if std:
            cfg.model.decoder.emb.param_noise = GaussianParameterNoise.default_config().set(std=std)
        trainer = cfg.instantiate(parent=None)
        return trainer.run(prng.PRNGKey(0))["loss"].item()

    assert run(0.0) != run(0.5)
