"""Orbax-protocol checkpointer: commit by rename / commit file, tracker file, retention, restore."""

import json
import os

import pytest
import torch

from axlearn_b200.common.checkpointer import every_n_steps_policy
from axlearn_b200.common.checkpointer_orbax import COMMIT_FILE, METADATA_FILE, TMP_MARKER, TRACKER_FILE, OrbaxCheckpointer
from axlearn_b200.common.config import config_for_function


def _state(seed):
    g = torch.Generator().manual_seed(seed)
    return {"model": {"w": torch.randn(6, 4, generator=g), "b": torch.randn(4, generator=g).bfloat16()},
            "learner": {"count": torch.tensor(seed)}, "prng_key": torch.tensor([seed, 7], dtype=torch.int64)}


def _ckpt(tmp_path, **kw):
    cfg = OrbaxCheckpointer.default_config().set(
        name="ckpt", dir=str(tmp_path), save_policy=config_for_function(every_n_steps_policy).set(n=2), **kw)
    return cfg.instantiate(parent=None)


def _zeros_like(tree):
    return {k: _zeros_like(v) if isinstance(v, dict) else torch.zeros_like(v) for k, v in tree.items()}


def _assert_equal(a, b):
    for k in a:
        if isinstance(a[k], dict):
            _assert_equal(a[k], b[k])
        else:
            assert a[k].dtype == b[k].dtype and torch.equal(a[k], b[k]), k


def test_save_commits_by_rename_and_restores(tmp_path):
    ck = _ckpt(tmp_path)
    assert not ck.save(step=1, state=_state(1))                   # the policy says no
    assert ck.save(step=2, state=_state(2))
    ck.wait_until_finished()
    names = sorted(os.listdir(tmp_path))
    assert names == [TRACKER_FILE, "step_00000002"], names        # no temporary directory is left
    step_dir = tmp_path / "step_00000002"
    assert sorted(os.listdir(step_dir)) == [METADATA_FILE, "index", "state"]
    meta = json.loads((step_dir / METADATA_FILE).read_text())
    assert meta["step"] == 2 and meta["commit_timestamp_nsecs"] >= meta["init_timestamp_nsecs"]
    entries = dict(json.loads((step_dir / "index" / "metadata").read_text()))
    assert entries["step"] == 2 and "model/w" in entries
    assert (tmp_path / TRACKER_FILE).read_text() == "step_00000002"
    assert OrbaxCheckpointer.checkpoint_steps(str(tmp_path)) == [2]
    step, restored = ck.restore(state=_zeros_like(_state(0)))
    assert step == 2
    _assert_equal(restored, _state(2))
    with pytest.raises(ValueError):
        ck.save(step=2, state=_state(2))                          # committed steps are never overwritten


def test_index_item_alone_is_not_a_commit(tmp_path):
    ck = _ckpt(tmp_path)
    half = tmp_path / f"step_00000004{TMP_MARKER}0"
    (half / "index").mkdir(parents=True)
    (half / "index" / "metadata").write_text("[]")
    inplace = tmp_path / "step_00000006"
    (inplace / "index").mkdir(parents=True)                        # final name, but nothing committed it
    assert OrbaxCheckpointer.checkpoint_paths(str(tmp_path)) == []
    assert ck.restore(state=_state(0))[0] is None
    # skip_uncommitted_checkpoint (default): the half-written step is left alone and not rewritten.
    assert not ck.save(step=4, state=_state(4))
    ck2 = _ckpt(tmp_path, skip_uncommitted_checkpoint=False, keep_last_n=2)
    assert ck2.save(step=4, state=_state(4)) and ck2.save(step=6, state=_state(6))
    ck2.wait_until_finished()
    assert OrbaxCheckpointer.checkpoint_steps(str(tmp_path)) == [4, 6]
    assert not half.exists()


def test_commit_file_protocol_for_stores_without_rename(tmp_path):
    ck = _ckpt(tmp_path, atomic_rename=False)
    assert ck.save(step=2, state=_state(2))
    ck.wait_until_finished()
    step_dir = tmp_path / "step_00000002"
    assert (step_dir / COMMIT_FILE).exists()
    os.remove(step_dir / COMMIT_FILE)                              # what a crash before the commit leaves
    assert OrbaxCheckpointer.checkpoint_steps(str(tmp_path)) == []
    with pytest.raises(ValueError):
        ck.restore(step=2, state=_state(0))


def test_retention_keeps_last_n_and_period(tmp_path):
    ck = _ckpt(tmp_path, keep_last_n=2, keep_period=4)
    for step in range(2, 16, 2):
        assert ck.save(step=step, state=_state(step))
        ck.wait_until_finished()
    assert OrbaxCheckpointer.checkpoint_steps(str(tmp_path)) == [4, 8, 12, 14]
    step, restored = ck.restore(step=8, state=_zeros_like(_state(0)))
    _assert_equal(restored, _state(8))


def test_tracker_file_selects_the_step(tmp_path):
    ck = _ckpt(tmp_path, keep_last_n=3, read_latest_checkpoint_from_tracker_file=True)
    for step in (2, 4):
        ck.save(step=step, state=_state(step))
        ck.wait_until_finished()
    (tmp_path / TRACKER_FILE).write_text("step_00000002")
    step, restored = ck.restore(state=_zeros_like(_state(0)))
    assert step == 2
    _assert_equal(restored, _state(2))
    (tmp_path / TRACKER_FILE).write_text("step_00000099")          # stale tracker: fall back to listing
    assert ck.restore(state=_zeros_like(_state(0)))[0] == 4
