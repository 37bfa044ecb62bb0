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


def test_delayed_scaling_state_lives_in_the_trainer_state(tmp_path):
    """Per-tensor delayed scaling: scale and amax-history parameters exist under the reference's
    names, are overwritten in place every step (never touched by the optimizer), and training
    tracks full precision."""
    from axlearn_b200.common.utils import flatten_items

    steps = 5
    kw = dict(max_step=steps, save_every_n_steps=1000, hidden=128, heads=1, ffn=256, vocab=512, seq=32, batch=8, layers=2)
    ref, _ = _losses(tiny_fuji_trainer_config(tmp_path / "ref", **kw), steps)
    cfg = tiny_fuji_trainer_config(tmp_path / "fp8t", **kw)
    cfg = FP8ConfigModifier.default_config().set(scaling="tensor", fp8_amax_history_length=4).instantiate()(cfg)
    got, trainer = _losses(cfg, steps)
    for a, b in zip(got, ref):
        assert abs(a - b) < 0.05 * abs(b), (got, ref)
    state = dict(flatten_items(trainer.trainer_state["model"]))
    base = "decoder/transformer/repeat/layer/feed_forward/linear2/quantized_dot_general/"
    for name in ("input_scale", "kernel_scale", "output_grad_scale"):
        v = state[base + name]
        assert v.shape == (2,) and v.dtype == torch.float32          # stacked over the 2 layers
        assert torch.all(v > 0) and not torch.allclose(v, torch.ones_like(v)), name
    hist = state[base + "input_amax_history"]
    assert hist.shape == (2, 4) and torch.all(hist > 0)              # 5 steps filled all 4 slots
    # Delayed scaling: the stored scale came from the history BEFORE this step's amax went in, so
    # it is at least (up to bf16 rounding of the working copy) the newest window's maximum / 448
    # whenever the slot that rolled out held the largest value, and of the same magnitude.
    want = hist.max(dim=1).values / 448.0
    scale = state[base + "input_scale"]
    assert torch.all(scale > 0.5 * want) and torch.all(scale < 2.0 * want)
    # No optimizer moments exist for the overridden parameters.
    opt = dict(flatten_items(trainer.trainer_state["learner"]))
    assert not any("amax_history" in p or p.endswith("_scale") for p in opt)
    assert any(p.endswith("linear2/weight") for p in opt)
