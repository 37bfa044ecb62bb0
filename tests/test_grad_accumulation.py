"""Gradient accumulation: N micro-batches per optimizer step reproduce the full-batch step."""

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.trainer_config_modifier import GradientAccumulationModifier
from tests.helpers import tiny_fuji_trainer_config


def _run(tmp, acc_steps):
    cfg = tiny_fuji_trainer_config(tmp, max_step=3, save_every_n_steps=100, hidden=32, heads=2, ffn=64, vocab=64,
                                   seq=16, batch=8, layers=2)
    if acc_steps > 1:
        cfg = GradientAccumulationModifier.default_config().set(grad_acc_steps=acc_steps).instantiate()(cfg)
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    data = iter(trainer.input.dataset())
    losses = [trainer.train_step(next(data))["loss"].item() for _ in range(3)]
    w = trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]["linear2"]["weight"]
    return losses, w.clone()


def test_accumulated_micro_batches_match_the_full_batch(tmp_path):
    full_losses, full_w = _run(tmp_path / "full", 1)
    acc_losses, acc_w = _run(tmp_path / "acc", 4)
    # Every micro-batch normalises by its own live-target count, so the match is close but not
    # bitwise (counts differ by the few targets that equal the padding id).
    for a, b in zip(acc_losses, full_losses):
        assert abs(a - b) < 2e-3 * abs(b), (acc_losses, full_losses)
    d = (acc_w - full_w).abs()
    # Adam normalises updates, so tiny gradient differences can move single elements by ~lr.
    assert d.mean() < 1e-4 and d.max() < 3e-3, (d.mean(), d.max())
