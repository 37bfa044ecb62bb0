"""The trainer refuses to keep or persist a step computed by a kernel that reported an error."""

import os

import pytest

from axlearn_b200.common import prng
from axlearn_b200.common.checkpointer import checkpoint_paths
from tests.helpers import tiny_fuji_trainer_config


def test_status_error_vetoes_the_checkpoint(tmp_path):
    cfg = tiny_fuji_trainer_config(tmp_path, max_step=4, save_every_n_steps=2, layers=1, vocab=256)
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    calls = {"n": 0}

    def fake_status_check():
        # Stands in for cuda_ops.check_status() finding a bounded-wait time-out code.
        calls["n"] += 1
        raise RuntimeError("device kernel reported status 4: gave up waiting for a peer flag")

    trainer._check_device_status = fake_status_check  # pylint: disable=protected-access
    with pytest.raises(RuntimeError, match="status 4"):
        trainer.save_checkpoint(force=True)
    assert calls["n"] == 1
    ckpt_dir = os.path.join(str(tmp_path), "checkpoints")
    assert not os.path.isdir(ckpt_dir) or checkpoint_paths(ckpt_dir) == []


def test_policy_that_declines_does_not_run_the_check(tmp_path):
    cfg = tiny_fuji_trainer_config(tmp_path, max_step=4, save_every_n_steps=100, layers=1, vocab=256)
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    trainer._step = 3  # pylint: disable=protected-access

    def boom():
        raise AssertionError("the check must only run when a checkpoint is about to be written")

    trainer._check_device_status = boom  # pylint: disable=protected-access
    assert trainer.save_checkpoint() is False


@pytest.mark.gpu
def test_unset_flag_wait_makes_trainer_refuse_to_checkpoint(tmp_path):
    """A wait on a flag that nothing sets runs out (bounded), leaves its code in the status word,
    and the trainer then refuses to write a checkpoint."""
    import torch

    from axlearn_b200.ops import cuda_ops, fused_comm

    cfg = tiny_fuji_trainer_config(tmp_path, max_step=4, save_every_n_steps=2, layers=1, vocab=256,
                                   device="cuda:0", train_dtype=torch.bfloat16)
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    fused_comm.wait_flags(flags, 2, 1)  # nothing sets these flags: the wait gives up after its poll budget
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status"):
        trainer.save_checkpoint(force=True)
    cuda_ops.check_status()  # cleared by the failed check above
    ckpt_dir = os.path.join(str(tmp_path), "checkpoints")
    assert not os.path.isdir(ckpt_dir) or checkpoint_paths(ckpt_dir) == []
