"""Goodput recording through a cloud goodput service.

Parity target: axlearn/cloud/gcp/measurement.py (``GoodputRecorder`` :38: maps framework events to
the calls of the ``ml-goodput-measurement`` recorder, uploads goodput / badput on an interval from
one process, optional rolling-window reporting).  That library is not in this image, so the
service is an interface (``GoodputClient``): a deployment injects the real client, tests a fake,
and without either the recorder writes the same events to a JSON-lines file that
``common.measurement.compute_goodput`` reads.
"""

from __future__ import annotations

import json
import os
import threading
import time
from typing import Any, Optional, Protocol, Sequence

from axlearn_b200.common import measurement
from axlearn_b200.common.config import config_class


class GoodputClient(Protocol):
    def record(self, event: str, *, timestamp: float, **fields) -> None: ...

    def upload(self, report: dict) -> None: ...


class _FileClient:
    def __init__(self, path: str):
        self._path = path
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self._lock = threading.Lock()

    def record(self, event: str, *, timestamp: float, **fields) -> None:
        with self._lock, open(self._path, "a", encoding="utf-8") as f:
            f.write(json.dumps({"event": event, "time": timestamp, **fields}) + "\n")

    def upload(self, report: dict) -> None:
        with self._lock, open(self._path + ".report", "w", encoding="utf-8") as f:
            json.dump(report, f)


@measurement.register_recorder("goodput")
class GoodputRecorder(measurement.Recorder):
    @config_class
    class Config(measurement.Recorder.Config):
        upload_dir: Optional[str] = None          # where the file fallback writes
        upload_interval: int = 30                 # seconds between reports
        rolling_window_size: Sequence[int] = ()   # seconds; one report per window size
        jax_backend: Optional[str] = None         # accepted for config parity; unused

    def __init__(self, cfg, *, client: Optional[GoodputClient] = None, process_index: int = 0):
        super().__init__(cfg)
        self._process_index = process_index
        self._client = client
        self._events: list = []
        self._monitor: Optional[threading.Thread] = None
        self._stop = threading.Event()

    def _get_client(self) -> GoodputClient:
        if self._client is None:
            cfg = self._config
            if cfg.upload_dir is None:
                raise ValueError("GoodputRecorder needs a client or an upload_dir")
            self._client = _FileClient(os.path.join(cfg.upload_dir, f"goodput_{cfg.name}.jsonl"))
        return self._client

    def record(self, event: measurement.Event, *args, **kwargs) -> None:
        now = time.time()
        fields = dict(kwargs)
        if event == measurement.Event.START_STEP and args:
            fields["step"] = int(args[0])
        # Every process records its own job start / end (needed to see stragglers); the other
        # events are recorded by the first process only.
        if self._process_index != 0 and event not in (measurement.Event.START_JOB, measurement.Event.END_JOB):
            return
        self._events.append({"event": event.value, "time": now, **fields})
        self._get_client().record(event.value, timestamp=now, process=self._process_index, **fields)

    def report(self, *, now: Optional[float] = None) -> dict:
        """Goodput over the whole job and over every rolling window."""
        now = time.time() if now is None else now
        out = {"job": measurement.compute_goodput(self._events, now=now)}
        for window in self._config.rolling_window_size:
            recent = [e for e in self._events if e["time"] >= now - window]
            out[f"window_{window}s"] = measurement.compute_goodput(recent, now=now) if recent else None
        return out

    def start_monitoring(self, **kwargs) -> None:
        if self._process_index != 0 or self._monitor is not None:
            return

        def loop():
            while not self._stop.wait(self._config.upload_interval):
                self._get_client().upload(self.report())

        self._monitor = threading.Thread(target=loop, daemon=True)
        self._monitor.start()

    def stop_monitoring(self) -> None:
        self._stop.set()
        if self._monitor is not None:
            self._monitor.join(timeout=5)
            self._monitor = None
        if self._process_index == 0 and self._events:
            self._get_client().upload(self.report())
