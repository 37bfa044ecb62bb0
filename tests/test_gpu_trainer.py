"""A small Fuji trained for a few steps on the GPU with the sm_100a kernels vs the same run on
PyTorch reference ops."""

import pytest
import torch

from axlearn_b200.common import prng
from tests.helpers import tiny_fuji_trainer_config

pytestmark = pytest.mark.gpu


def _losses(tmp_path, name, reference_ops: bool, steps=4):
    from axlearn_b200.ops import dispatch

    cfg = tiny_fuji_trainer_config(
        tmp_path / name, max_step=steps, save_every_n_steps=1000, train_dtype=torch.bfloat16, device="cuda",
        hidden=256, heads=2, ffn=512, vocab=4096, seq=256, batch=4, layers=2, scan_chunk=512, shared_lm_head=True)
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    losses = []
    it = iter(trainer.input.dataset())
    for _ in range(steps):
        if reference_ops:
            with dispatch.use_reference_ops():
                out = trainer.train_step(next(it))
        else:
            out = trainer.train_step(next(it))
        losses.append(out["loss"].item())
    return losses


def test_kernel_path_tracks_reference_path(tmp_path):
    from axlearn_b200.ops import cuda_ops

    fast = _losses(tmp_path, "fast", reference_ops=False)
    cuda_ops.check_status()
    slow = _losses(tmp_path, "slow", reference_ops=True)
    for a, b in zip(fast, slow):
        assert abs(a - b) < 2e-2 * abs(b), (fast, slow)
    assert cuda_ops.launch_count > 0
