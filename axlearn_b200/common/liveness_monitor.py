"""Liveness of a training job judged from the outside, by the age of its newest summary file.

Parity target in the reference: ``LivenessMonitor`` (axlearn/common/liveness_monitor.py:33-109):
launchers poll ``ping()``; a job whose summary directory has not changed for
``max_timeout_seconds`` (``max_start_seconds`` before the first file appears) is declared dead.
"""

from __future__ import annotations

import os
import time
from typing import Optional

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class


class LivenessMonitor(Configurable):
    @config_class
    class Config(Configurable.Config):
        summary_dir: Required[str] = REQUIRED
        max_timeout_seconds: float = 3600.0
        max_start_seconds: float = 7200.0

    def __init__(self, cfg):
        super().__init__(cfg)
        self._started_at: Optional[float] = None
        self._latest_mtime: Optional[float] = None

    def started(self) -> bool:
        return self._started_at is not None

    def reset(self) -> None:
        self._started_at = time.time()
        self._latest_mtime = None

    def _newest_mtime(self) -> Optional[float]:
        newest = None
        for root, _, files in os.walk(self._config.summary_dir):
            for f in files:
                try:
                    m = os.path.getmtime(os.path.join(root, f))
                except OSError:
                    continue
                newest = m if newest is None else max(newest, m)
        return newest

    def ping(self) -> bool:
        """True while the job looks alive."""
        if self._started_at is None:
            raise RuntimeError("call reset() when the job starts")
        cfg = self._config
        now = time.time()
        newest = self._newest_mtime()
        if newest is None:
            return now - self._started_at <= cfg.max_start_seconds
        self._latest_mtime = newest
        return now - max(newest, self._started_at) <= cfg.max_timeout_seconds
