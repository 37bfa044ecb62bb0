"""Jobs: units of work with retries.

Parity target in the reference: axlearn/cloud/common/job.py (``Job`` with ``_execute`` /
``execute`` retry loop, ``_delete``).
"""

from __future__ import annotations

import logging
import subprocess
import time
from typing import Any, Optional

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class


class Job(Configurable):
    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED
        max_tries: int = 1
        retry_interval: float = 1.0
        command: Optional[str] = None

    def _delete(self) -> None:
        """Releases whatever the job holds; must be idempotent."""

    def _execute(self) -> Any:
        cfg = self._config
        if cfg.command is None:
            raise NotImplementedError(type(self))
        return subprocess.run(cfg.command, shell=True, check=True).returncode

    def execute(self) -> Any:
        cfg = self._config
        tries = 0
        while True:
            tries += 1
            try:
                return self._execute()
            except Exception as e:  # pylint: disable=broad-except
                logging.warning("job %s failed (try %d of %d): %s", cfg.name, tries, cfg.max_tries, e)
                if tries >= cfg.max_tries:
                    self._delete()
                    raise
                time.sleep(cfg.retry_interval)
