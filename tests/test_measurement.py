"""Goodput recorder: event log, report arithmetic, trainer integration."""

import json

import pytest

from axlearn_b200.common import measurement
from axlearn_b200.common.measurement import Event, EventType, FileRecorder, compute_goodput, read_events


def test_compute_goodput_with_restart_and_overheads():
    ev = lambda name, t, **kw: {"event": name, "time": float(t), **kw}
    events = [
        ev("START_JOB", 0), ev("START_TRAINING_PREPARATION", 0), ev("END_TRAINING_PREPARATION", 10),
        ev("START_DATA_LOADING", 10), ev("END_DATA_LOADING", 12),
        ev("START_STEP", 12, step=1), ev("START_DATA_LOADING", 20), ev("END_DATA_LOADING", 21),
        ev("START_STEP", 21, step=2),                       # crashes at t = 30: no END_JOB
        ev("START_JOB", 40), ev("START_TRAINING_PREPARATION", 40), ev("END_TRAINING_PREPARATION", 45),
        ev("START_STEP", 45, step=2), ev("START_STEP", 55, step=3), ev("END_JOB", 65),
    ]
    r = compute_goodput(events)
    assert r["total_seconds"] == 65
    # step 1: 12 -> 21 minus 1 s of data loading = 8; step 2 (second run): 10; step 3: 10.
    assert r["productive_seconds"] == pytest.approx(28)
    assert r["badput"]["wasted_progress"] == pytest.approx(19)        # first run of step 2: 21 -> 40
    assert r["badput"]["training_preparation"] == pytest.approx(15)
    assert r["badput"]["data_loading"] == pytest.approx(3)
    assert r["goodput"] == pytest.approx(28 / 65)
    assert sum(r["badput"].values()) + r["productive_seconds"] == pytest.approx(65)
    assert compute_goodput([])["goodput"] == 0.0


def test_file_recorder_and_registry(tmp_path):
    cfg = measurement.get_recorder_config("file", [f"dir={tmp_path}", "report_interval_seconds=0"])
    rec = cfg.instantiate()
    assert isinstance(rec, FileRecorder)
    rec.record(Event.START_JOB)
    with rec.record_event(EventType.ACCELERATOR_INIT):
        pass
    with rec.record_event(EventType.STEP, 7):
        pass
    rows = read_events(rec.path)
    assert [r["event"] for r in rows] == ["START_JOB", "START_ACCELERATOR_INIT", "END_ACCELERATOR_INIT", "START_STEP"]
    assert rows[-1]["step"] == 7
    with pytest.raises(NotImplementedError):
        measurement.get_recorder_config("nope")
    with pytest.raises(ValueError):
        measurement.register_recorder("file")(FileRecorder)


def test_trainer_records_goodput_events(tmp_path):
    from axlearn_b200.common import prng
    from tests.helpers import tiny_fuji_trainer_config

    cfg = tiny_fuji_trainer_config(str(tmp_path / "run"), max_step=3, save_every_n_steps=100)
    cfg.recorder = FileRecorder.default_config().set(dir=str(tmp_path / "goodput"))
    trainer = cfg.instantiate(parent=None)
    trainer.run(prng.PRNGKey(0))
    rows = read_events(str(tmp_path / "goodput" / "goodput_events.jsonl"))
    names = [r["event"] for r in rows]
    assert names[0] == "START_JOB" and names[-1] == "END_JOB"
    assert names.count("START_STEP") == 3 and [r["step"] for r in rows if r["event"] == "START_STEP"] == [1, 2, 3]
    assert names.index("END_TRAINING_PREPARATION") < names.index("START_STEP")
    report = compute_goodput(rows)
    assert 0 < report["goodput"] <= 1
    json.dumps(report)
