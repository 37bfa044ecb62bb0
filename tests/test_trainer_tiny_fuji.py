"""The smallest benchmark config on CPU: 20 trainer steps of a tiny Fuji, checkpoint, restore, bit-match."""

import json
import os

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.checkpointer import checkpoint_paths, read_index_file
from axlearn_b200.common.utils import flatten_items
from tests.helpers import tiny_fuji_trainer_config


def _run(directory, max_step, *, stop_after=None):
    cfg = tiny_fuji_trainer_config(directory, max_step=max_step)
    cfg.save_input_iterator = True
    if stop_after is not None:
        # The input runs dry after `stop_after` batches: the run ends early, as if interrupted.
        cfg.input.total_num_batches = stop_after
    trainer = cfg.instantiate(parent=None)
    out = trainer.run(prng.PRNGKey(0))
    return trainer, out


def test_train_20_steps_and_resume_bit_match(tmp_path):
    full, out_full = _run(tmp_path / "full", 20)
    assert full.step == 20
    loss_full = out_full["loss"].item()
    assert abs(loss_full - 10.397) < 0.2  # ~ln(32768) on uniform random tokens

    # Same run interrupted at step 10 (checkpoint saved there), resumed by a new trainer.
    first, _ = _run(tmp_path / "resume", 20, stop_after=10)
    assert first.step == 10
    assert [os.path.basename(p) for p in checkpoint_paths(str(tmp_path / "resume" / "checkpoints"))] == ["step_00000010"]
    second, out_resumed = _run(tmp_path / "resume", 20)
    assert second.step == 20
    assert out_resumed["loss"].item() == loss_full  # bit-exact
    for (pa, a), (pb, b) in zip(flatten_items(full.trainer_state), flatten_items(second.trainer_state)):
        assert pa == pb
        assert torch.equal(a.cpu(), b.cpu()), pa


def test_checkpoint_layout_and_names(tmp_path):
    trainer, _ = _run(tmp_path / "run", 10)
    ckpt = tmp_path / "run" / "checkpoints" / "step_00000010"
    index = read_index_file(str(ckpt))
    assert index[0] == ("step", 10)
    entries = dict(index)
    qkv = "model/decoder/transformer/repeat/layer/self_attention/attention/i_proj/i_proj/qkv_proj/weight"
    assert entries[qkv] == {"dtype": "float32", "shape": "(4, 3, 128, 4, 32)"}
    assert entries["prng_key"] == {"dtype": "uint32", "shape": "(4,)"}
    # Optimizer leaves follow the chain nesting: chain(clip, chain(adam, lr, wd, update, neg)).
    assert entries["learner/optimizer/1/0/count"] == {"dtype": "int32", "shape": "()"}
    assert f"learner/optimizer/1/0/mu/{qkv[len('model/'):]}" in entries
    assert f"learner/optimizer/1/0/nu/{qkv[len('model/'):]}" in entries
    assert "learner/optimizer/1/1/count" in entries and "learner/optimizer/1/3/count" in entries
    assert not any(k.startswith("learner/optimizer/0") for k in entries)
    # One zarr array per leaf with a single chunk named by shard coordinates.
    adir = ckpt / "gda" / qkv
    meta = json.loads((adir / ".zarray").read_text())
    assert meta["shape"] == [4, 3, 128, 4, 32] and meta["chunks"] == [4, 3, 128, 4, 32]
    assert (adir / "0.0.0.0.0").stat().st_size == 4 * 3 * 128 * 4 * 32 * 4
    assert (ckpt / "gda" / "learner/optimizer/1/0/count" / "0").exists()
    # An uncommitted directory (no index) is ignored.
    os.remove(ckpt / "index")
    assert checkpoint_paths(str(tmp_path / "run" / "checkpoints")) == []
