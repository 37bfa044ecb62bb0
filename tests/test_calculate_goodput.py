"""Goodput daemon (reference behaviour: axlearn/experiments/calculate_goodput.py)."""

import json

from axlearn_b200.experiments import calculate_goodput as cg


def _write_events(path):
    events = [("START_JOB", 0.0, {}), ("START_ACCELERATOR_INIT", 0.0, {}), ("END_ACCELERATOR_INIT", 10.0, {}),
              ("START_STEP", 10.0, {"step": 1}), ("START_STEP", 40.0, {"step": 2}), ("END_JOB", 100.0, {})]
    with open(path, "w", encoding="utf-8") as f:
        for name, t, extra in events:
            f.write(json.dumps({"event": name, "time": t, **extra}) + "\n")


def test_bodies_follow_the_monitoring_api():
    d = cg.metric_descriptor_body()
    assert d["type"] == "custom.googleapis.com/goodput" and d["metricKind"] == "GAUGE" and d["valueType"] == "DOUBLE"
    body = cg.time_series_body(value=87.5, resource_labels={"location": "us-x"}, metric_labels={"job_name": "j"},
                               end_time=1_700_000_000.0)
    (ts,) = body["timeSeries"]
    assert ts["resource"] == {"type": "generic_node", "labels": {"namespace": "namespace", "node_id": "node_id", "location": "us-x"}}
    assert ts["metric"]["labels"]["goodput"] == "87.5" and ts["metric"]["labels"]["job_name"] == "j"
    assert ts["metric"]["labels"]["event_time"] == "14 Nov 2023 22:13:20 UTC"
    assert ts["points"] == [{"interval": {"endTime": "2023-11-14T22:13:20Z"}, "value": {"doubleValue": 87.5}}]


def test_report_once_and_daemon(tmp_path, capsys):
    events = str(tmp_path / "events.jsonl")
    _write_events(events)
    published = []
    out = cg.report_once(job_name="j", events_path=events, zone="z", now=100.0, publish=published.append,
                         output=str(tmp_path / "readings.jsonl"))
    assert abs(out["goodput_percent"] - 90.0) < 1e-6 and out["badput"]["accelerator_init"] == 10.0
    assert published[0]["timeSeries"][0]["points"][0]["value"]["doubleValue"] == out["goodput_percent"]
    line = json.loads(open(tmp_path / "readings.jsonl", encoding="utf-8").read())
    assert line["job_name"] == "j" and "time_series" not in line

    naps = []
    n = cg.main(["--job_name", "j", "--events", events, "--interval", "5", "--max_readings", "3"],
                publish=published.append, sleep=naps.append)
    assert n == 3 and naps == [5.0, 5.0] and len(published) == 4
    assert "Job goodput: 90.0000%" in capsys.readouterr().out
    assert cg.main(["--job_name", "j", "--events", str(tmp_path / "missing.jsonl")]) == 1
