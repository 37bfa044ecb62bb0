"""Job lifecycle events published by the bastion.

Counterpart of axlearn/cloud/common/event_queue.py (``Event``, ``BaseQueueClient``,
``RabbitMQClient``).  The bastion emits one event per job state change; a queue client delivers
them.  Built here: a client that appends JSON lines to a file of the shared directory (the
transport that fits a bastion coordinating through a shared directory) and an in-memory client for
tests; a message-broker client plugs in by implementing ``publish``.
"""

from __future__ import annotations

import dataclasses
import json
import os
import threading
import time
from typing import Optional


@dataclasses.dataclass
class JobLifecycleEvent:
    job_name: str
    state: str                       # PENDING / ACTIVE / CLEANING / COMPLETED ...
    details: str = ""
    job_id: Optional[str] = None
    timestamp: float = 0.0

    def serialize(self) -> str:
        d = dataclasses.asdict(self)
        d["timestamp"] = d["timestamp"] or time.time()
        return json.dumps(d, sort_keys=True)


class BaseQueueClient:
    def publish(self, event: JobLifecycleEvent) -> None:
        raise NotImplementedError(type(self))

    def close(self) -> None:
        pass


class InMemoryQueueClient(BaseQueueClient):
    def __init__(self):
        self.events: list[JobLifecycleEvent] = []

    def publish(self, event):
        self.events.append(event)


class FileQueueClient(BaseQueueClient):
    """Appends to ``path``; every line is written with one ``os.write`` on an ``O_APPEND``
    descriptor, so that concurrent publishers never interleave inside a line.  Failures to publish
    are counted, not raised: events are advisory and must not take the scheduler down."""

    def __init__(self, path: str, *, num_tries: int = 2):
        self._path, self._tries = path, num_tries
        self._lock = threading.Lock()
        self.dropped = 0
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def publish(self, event):
        line = (event.serialize() + "\n").encode()
        with self._lock:
            for _ in range(self._tries):
                try:
                    fd = os.open(self._path, os.O_WRONLY | os.O_APPEND | os.O_CREAT, 0o644)
                    try:
                        os.write(fd, line)
                    finally:
                        os.close(fd)
                    return
                except OSError:
                    time.sleep(0.01)
            self.dropped += 1

    def read_all(self) -> list[dict]:
        if not os.path.exists(self._path):
            return []
        with open(self._path) as f:
            return [json.loads(line) for line in f if line.strip()]
