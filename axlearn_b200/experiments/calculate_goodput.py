"""Computes a job's goodput from its event log and publishes it (reference:
axlearn/experiments/calculate_goodput.py).

    python -m axlearn_b200.experiments.calculate_goodput --job_name my-job --events /runs/my-job/goodput.jsonl
    python -m axlearn_b200.experiments.calculate_goodput --job_name my-job --events ... --interval 300   # daemon

The reference asks the ``ml_goodput_measurement`` service for the figure and writes it to Cloud
Monitoring as the custom gauge ``custom.googleapis.com/goodput`` on a ``generic_node`` resource.
Here the figure comes from the event file that ``measurement.FileRecorder`` /
``cloud.gcp.measurement.GoodputRecorder`` append to.  The Cloud Monitoring requests are built as
plain dictionaries (``metric_descriptor_body`` / ``time_series_body``) and handed to a ``publish``
callable, so a deployment can pass its own authorised client; without one the report is printed and,
with ``--output``, appended to a JSON Lines file.
"""

from __future__ import annotations

import argparse
import json
import time
from datetime import datetime, timezone
from typing import Callable, Optional, Sequence

from axlearn_b200.common import measurement

METRIC_NAME = "goodput"


def metric_descriptor_body(metric_name: str = METRIC_NAME) -> dict:
    """Body of ``projects.metricDescriptors.create`` for the gauge."""
    return {"name": metric_name, "type": f"custom.googleapis.com/{metric_name}",
            "description": f"{metric_name.capitalize()} metric.", "displayName": metric_name.capitalize(),
            "metricKind": "GAUGE", "valueType": "DOUBLE"}


def time_series_body(*, metric_name: str = METRIC_NAME, value: float, resource_labels: dict, metric_labels: dict,
                     end_time: float) -> dict:
    """Body of ``projects.timeSeries.create`` with one point at ``end_time`` (seconds since the epoch)."""
    utc = datetime.fromtimestamp(end_time, tz=timezone.utc)
    return {"timeSeries": [{
        "metric": {"type": f"custom.googleapis.com/{metric_name}",
                   "labels": {metric_name: str(value), "event_time": utc.strftime("%d %b %Y %H:%M:%S UTC"),
                              **metric_labels}},
        # The namespace / node_id labels are mandatory for a generic_node.
        "resource": {"type": "generic_node", "labels": {"namespace": "namespace", "node_id": "node_id", **resource_labels}},
        "points": [{"interval": {"endTime": utc.strftime("%Y-%m-%dT%H:%M:%SZ")}, "value": {"doubleValue": value}}],
    }]}


def report_once(*, job_name: str, events_path: str, zone: str = "", now: Optional[float] = None,
                publish: Optional[Callable[[dict], None]] = None, output: Optional[str] = None) -> dict:
    """One reading: goodput in percent (as the reference prints it), the badput breakdown, and the
    time-series body that was published."""
    start = time.time()
    report = measurement.compute_goodput(measurement.read_events(events_path), now=now)
    end = now if now is not None else time.time()
    percent = 100.0 * report["goodput"]
    body = time_series_body(value=percent, resource_labels={"location": zone}, metric_labels={"job_name": job_name},
                            end_time=end)
    if publish is not None:
        publish(body)
    out = {"job_name": job_name, "goodput_percent": percent, "fetch_seconds": time.time() - start, **report,
           "time_series": body}
    if output:
        with open(output, "a", encoding="utf-8") as f:
            f.write(json.dumps({k: v for k, v in out.items() if k != "time_series"}) + "\n")
    return out


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__.split("\n", 1)[0])
    ap.add_argument("--job_name", required=True)
    ap.add_argument("--events", required=True, help="Event file written by the job's goodput recorder.")
    ap.add_argument("--zone", default="")
    ap.add_argument("--output", default=None, help="Append each reading to this JSON Lines file.")
    ap.add_argument("--interval", type=float, default=0.0, help="Seconds between readings; 0 = one reading.")
    ap.add_argument("--max_readings", type=int, default=0, help="Stop after this many readings (0 = never).")
    return ap


def main(argv: Optional[Sequence[str]] = None, *, publish: Optional[Callable[[dict], None]] = None,
         sleep: Callable[[float], None] = time.sleep) -> int:
    args = parser().parse_args(argv)
    n = 0
    while True:
        out = report_once(job_name=args.job_name, events_path=args.events, zone=args.zone, publish=publish,
                          output=args.output)
        n += 1
        print(f"Job goodput: {out['goodput_percent']:.4f}%")
        print(f"Fetch time: {out['fetch_seconds']:.2f} seconds")
        for category, seconds in sorted(out["badput"].items()):
            print(f"  badput/{category}: {seconds:.1f} s")
        if args.interval <= 0 or (args.max_readings and n >= args.max_readings):
            return n
        sleep(args.interval)


if __name__ == "__main__":
    main()
