"""Goodput measurement: recording job events and computing productive-time fractions.

Parity targets in the reference: ``Event`` / ``EventType`` / ``Recorder`` / ``register_recorder``
/ ``define_flags`` (axlearn/common/measurement_base.py:13-164), the module-level
``initialize`` / ``record_event`` / ``start_monitoring`` (axlearn/common/measurement.py) and the
cloud implementation's semantics (axlearn/cloud/gcp/measurement.py: events appended to a durable
log, goodput = productive training time / wall time with badput split by cause).

``FileRecorder`` appends JSON lines ``{"event", "time", "step"?, ...}`` to
``<dir>/goodput_events.jsonl`` (rank 0 only by default); ``compute_goodput`` turns such a log --
possibly spanning several restarts of the job -- into a report.  Step time counts as productive
only up to the last step that was not lost: steps redone after a restart are badput
("wasted progress").
"""

from __future__ import annotations

import contextlib
import enum
import json
import os
import threading
import time
from typing import Any, Optional, Sequence

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class


class Event(enum.Enum):
    START_JOB = "START_JOB"
    END_JOB = "END_JOB"
    START_STEP = "START_STEP"
    START_ACCELERATOR_INIT = "START_ACCELERATOR_INIT"
    END_ACCELERATOR_INIT = "END_ACCELERATOR_INIT"
    START_TRAINING_PREPARATION = "START_TRAINING_PREPARATION"
    END_TRAINING_PREPARATION = "END_TRAINING_PREPARATION"
    START_DATA_LOADING = "START_DATA_LOADING"
    END_DATA_LOADING = "END_DATA_LOADING"
    START_CUSTOM_BADPUT_EVENT = "START_CUSTOM_BADPUT_EVENT"
    END_CUSTOM_BADPUT_EVENT = "END_CUSTOM_BADPUT_EVENT"


class EventType(enum.Enum):
    JOB = "job"
    STEP = "step"
    ACCELERATOR_INIT = "accelerator_init"
    TRAINING_PREPARATION = "training_preparation"
    DATA_LOADING = "data_loading"
    CUSTOM_BADPUT_EVENT = "custom_badput_event"


_START_END = {
    EventType.JOB: (Event.START_JOB, Event.END_JOB),
    EventType.ACCELERATOR_INIT: (Event.START_ACCELERATOR_INIT, Event.END_ACCELERATOR_INIT),
    EventType.TRAINING_PREPARATION: (Event.START_TRAINING_PREPARATION, Event.END_TRAINING_PREPARATION),
    EventType.DATA_LOADING: (Event.START_DATA_LOADING, Event.END_DATA_LOADING),
    EventType.CUSTOM_BADPUT_EVENT: (Event.START_CUSTOM_BADPUT_EVENT, Event.END_CUSTOM_BADPUT_EVENT),
}


class Recorder(Configurable):
    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED

    def record(self, event: Event, *args, **kwargs) -> None:
        raise NotImplementedError(type(self))

    def start_monitoring(self, **kwargs) -> None:
        """Starts whatever background reporting the recorder offers (none by default)."""

    @contextlib.contextmanager
    def record_event(self, event: EventType, *args, **kwargs):
        """Context manager recording the start / end pair of ``event`` (``STEP`` has only a start)."""
        if event == EventType.STEP:
            self.record(Event.START_STEP, *args, **kwargs)
            yield
            return
        start, end = _START_END[event]
        self.record(start, *args, **kwargs)
        try:
            yield
        finally:
            self.record(end, *args, **kwargs)


_recorders: dict[str, type] = {}


def register_recorder(name: str):
    def fn(cls):
        if name in _recorders:
            raise ValueError(f"recorder {name!r} is registered already")
        _recorders[name] = cls
        return cls

    return fn


def get_recorder_config(recorder_type: str, spec: Sequence[str] = ()) -> Recorder.Config:
    """``spec``: ``key=value`` strings applied to the recorder's config."""
    if recorder_type not in _recorders:
        raise NotImplementedError(f"unknown recorder type {recorder_type!r}; known: {sorted(_recorders)}")
    cfg = _recorders[recorder_type].default_config()
    for item in spec:
        k, _, v = item.partition("=")
        current = getattr(cfg, k)
        setattr(cfg, k, type(current)(v) if isinstance(current, (int, float)) and not isinstance(current, bool) else v)
    return cfg


@register_recorder("file")
class FileRecorder(Recorder):
    @config_class
    class Config(Recorder.Config):
        name: str = "file"
        dir: Required[str] = REQUIRED
        # Only this process index writes (events of the other ranks are the same to within noise).
        process_index: int = 0
        # start_monitoring() logs a goodput report this often (seconds); 0 = never.
        report_interval_seconds: float = 0.0

    def __init__(self, cfg):
        super().__init__(cfg)
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()

    @property
    def path(self) -> str:
        return os.path.join(self._config.dir, "goodput_events.jsonl")

    def _is_writer(self) -> bool:
        return int(os.environ.get("RANK", "0")) == self._config.process_index

    def record(self, event: Event, *args, **kwargs) -> None:
        if not self._is_writer():
            return
        row = {"event": event.value, "time": time.time()}
        if args:
            row["step"] = int(args[0])
        row.update({k: v for k, v in kwargs.items() if isinstance(v, (int, float, str, bool))})
        with self._lock:
            os.makedirs(self._config.dir, exist_ok=True)
            with open(self.path, "a", encoding="utf-8") as f:
                f.write(json.dumps(row) + "\n")

    def start_monitoring(self, **kwargs) -> None:
        interval = self._config.report_interval_seconds
        if interval <= 0 or self._thread is not None or not self._is_writer():
            return

        def loop():
            import logging

            while not self._stop.wait(interval):
                logging.info("goodput: %s", json.dumps(compute_goodput(read_events(self.path))))

        self._thread = threading.Thread(target=loop, name="goodput_monitor", daemon=True)
        self._thread.start()

    def stop_monitoring(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None


def read_events(path: str) -> list[dict]:
    if not os.path.exists(path):
        return []
    with open(path, encoding="utf-8") as f:
        return [json.loads(line) for line in f if line.strip()]


def compute_goodput(events: Sequence[dict], *, now: Optional[float] = None) -> dict:
    """``{"goodput", "total_seconds", "productive_seconds", "badput": {category: seconds}}``.

    Productive time = for every step number, the duration of its *last* execution (from its
    ``START_STEP`` to the next event); earlier executions of a step that was repeated after a
    restart are "wasted_progress".  Initialisation, preparation, data loading and custom
    intervals are their own categories; the rest ("other") is time between jobs and unexplained
    gaps."""
    events = sorted(events, key=lambda e: e["time"])
    if not events:
        return {"goodput": 0.0, "total_seconds": 0.0, "productive_seconds": 0.0, "badput": {}}
    end_time = now if now is not None else events[-1]["time"]
    total = max(0.0, end_time - events[0]["time"])
    badput = {"accelerator_init": 0.0, "training_preparation": 0.0, "data_loading": 0.0,
              "custom_badput_event": 0.0, "wasted_progress": 0.0}
    open_at: dict[str, float] = {}
    pairs = {"START_ACCELERATOR_INIT": ("END_ACCELERATOR_INIT", "accelerator_init"),
             "START_TRAINING_PREPARATION": ("END_TRAINING_PREPARATION", "training_preparation"),
             "START_DATA_LOADING": ("END_DATA_LOADING", "data_loading"),
             "START_CUSTOM_BADPUT_EVENT": ("END_CUSTOM_BADPUT_EVENT", "custom_badput_event")}
    ends = {end: (start, cat) for start, (end, cat) in pairs.items()}
    step_runs: dict[int, list[float]] = {}
    data_in_step = 0.0
    for i, e in enumerate(events):
        name = e["event"]
        if name in pairs:
            open_at[name] = e["time"]
        elif name in ends:
            start, cat = ends[name]
            if start in open_at:
                badput[cat] += e["time"] - open_at.pop(start)
        elif name == "START_STEP":
            # A step lasts until the next step start, job end or job start (a restart).
            nxt = end_time
            inner_data = 0.0
            data_open = None
            for later in events[i + 1:]:
                if later["event"] in ("START_STEP", "END_JOB", "START_JOB"):
                    nxt = later["time"]
                    break
                if later["event"] == "START_DATA_LOADING":
                    data_open = later["time"]
                elif later["event"] == "END_DATA_LOADING" and data_open is not None:
                    inner_data += later["time"] - data_open
                    data_open = None
            step_runs.setdefault(int(e.get("step", -1)), []).append(max(0.0, nxt - e["time"] - inner_data))
            data_in_step += inner_data
    productive = 0.0
    for runs in step_runs.values():
        productive += runs[-1]
        badput["wasted_progress"] += sum(runs[:-1])
    explained = productive + sum(badput.values())
    badput["other"] = max(0.0, total - explained)
    return {"goodput": productive / total if total > 0 else 0.0, "total_seconds": total,
            "productive_seconds": productive, "badput": badput}


# ------------------------------------------------------------------------------------------
# Process-wide recorder, as used by launchers.
# ------------------------------------------------------------------------------------------

global_recorder: Optional[Recorder] = None


def initialize(recorder_type: Optional[str], spec: Sequence[str] = ()) -> None:
    global global_recorder
    if global_recorder is not None or not recorder_type:
        return
    global_recorder = get_recorder_config(recorder_type, spec).instantiate()


def record_event(event: Event, *args, **kwargs) -> None:
    if global_recorder is not None:
        global_recorder.record(event, *args, **kwargs)


def start_monitoring(**kwargs) -> None:
    if global_recorder is not None:
        global_recorder.start_monitoring(**kwargs)
