"""Elastic replica state between a bastion and an external store (reference:
axlearn/cloud/common/replica_manager.py).

Once per scheduling cycle the bastion calls ``refresh()`` (optional bulk prefetch), asks
``get_desired_replicas(job)`` for every elastic job before scheduling, and reports
``set_granted_replicas(job, ...)`` for every elastic verdict afterwards.  ``FileReplicaManager`` keeps
the state as one JSON file per job in a directory -- the store a single-node deployment or a test
needs; a cluster deployment implements the same three methods over its own store.
"""

from __future__ import annotations

import json
import os
from typing import Mapping, Optional

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class

DESIRED_REPLICAS_KEY = "desired_replicas"
GRANTED_REPLICAS_KEY = "granted_replicas"


class ReplicaManager(Configurable):
    @config_class
    class Config(Configurable.Config):
        pass

    def refresh(self) -> None:
        """Prefetch hook, once per scheduling cycle."""

    def get_desired_replicas(self, job_name: str) -> Optional[Mapping[str, int]]:
        """``{scaling group: desired replicas}``, or None when the manager knows nothing of the job
        (the scheduler then uses the spec's ``min_replicas``)."""
        raise NotImplementedError(type(self))

    def set_granted_replicas(self, job_name: str, granted_replicas: Mapping[str, int]) -> None:
        raise NotImplementedError(type(self))


class FileReplicaManager(ReplicaManager):
    """``{root_dir}/{job}.json`` holding ``{"desired_replicas": {...}, "granted_replicas": {...}}``."""

    @config_class
    class Config(ReplicaManager.Config):
        root_dir: Required[str] = REQUIRED

    def __init__(self, cfg):
        super().__init__(cfg)
        os.makedirs(self._config.root_dir, exist_ok=True)
        self._cache: dict = {}

    def _path(self, job_name: str) -> str:
        return os.path.join(self._config.root_dir, f"{job_name}.json")

    def refresh(self) -> None:
        self._cache = {}
        for name in os.listdir(self._config.root_dir):
            if name.endswith(".json"):
                try:
                    with open(os.path.join(self._config.root_dir, name), encoding="utf-8") as f:
                        self._cache[name[:-5]] = json.load(f)
                except (OSError, ValueError):
                    continue                     # a file being written: next cycle sees it

    def _read(self, job_name: str) -> Optional[dict]:
        if job_name in self._cache:
            return self._cache[job_name]
        try:
            with open(self._path(job_name), encoding="utf-8") as f:
                return json.load(f)
        except (OSError, ValueError):
            return None

    def get_desired_replicas(self, job_name: str) -> Optional[Mapping[str, int]]:
        state = self._read(job_name)
        return None if state is None else state.get(DESIRED_REPLICAS_KEY)

    def set_desired_replicas(self, job_name: str, desired_replicas: Mapping[str, int]) -> None:
        """What an autoscaler (or an operator) writes."""
        self._write(job_name, DESIRED_REPLICAS_KEY, desired_replicas)

    def set_granted_replicas(self, job_name: str, granted_replicas: Mapping[str, int]) -> None:
        self._write(job_name, GRANTED_REPLICAS_KEY, granted_replicas)

    def get_granted_replicas(self, job_name: str) -> Optional[Mapping[str, int]]:
        state = self._read(job_name)
        return None if state is None else state.get(GRANTED_REPLICAS_KEY)

    def _write(self, job_name: str, key: str, value: Mapping[str, int]) -> None:
        state = dict(self._read(job_name) or {})
        state[key] = {k: int(v) for k, v in value.items()}
        tmp = self._path(job_name) + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            json.dump(state, f)
        os.replace(tmp, self._path(job_name))
        self._cache[job_name] = state
