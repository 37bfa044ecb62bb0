"""FP8ConfigModifier: the tiny Fuji trains with block-scaled fp8 projections and tracks the
full-precision loss curve."""

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.trainer_config_modifier import FP8ConfigModifier
from tests.helpers import tiny_fuji_trainer_config


def _losses(cfg, steps):
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    data = iter(trainer.input.dataset())
    return [trainer.train_step(next(data))["loss"].item() for _ in range(steps)], trainer


def test_fp8_training_tracks_full_precision(tmp_path):
    steps = 6
    kw = dict(max_step=steps, save_every_n_steps=1000, hidden=128, heads=1, ffn=256, vocab=512, seq=32, batch=8, layers=2)
    ref, _ = _losses(tiny_fuji_trainer_config(tmp_path / "ref", **kw), steps)
    cfg = tiny_fuji_trainer_config(tmp_path / "fp8", **kw)
    cfg = FP8ConfigModifier.default_config().set(scaling="block").instantiate()(cfg)
    got, trainer = _losses(cfg, steps)
    # The modifier reached the dense layers.
    layer = trainer.model.decoder.transformer.repeat.layer
    assert "quantized_dot_general" in layer.feed_forward.linear2.children
    assert ref[0] > ref[-1]                       # the reference itself learns
    for a, b in zip(got, ref):
        assert abs(a - b) < 0.03 * abs(b), (got, ref)
    assert got != ref                             # and fp8 rounding is really in the loop
