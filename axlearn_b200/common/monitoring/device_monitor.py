"""Device utilisation monitoring used by the trainer watchdog.

Parity targets in the reference: ``DeviceMonitorClient`` / ``DeviceMonitor``
(axlearn/common/monitoring/device_monitor.py:41-119): a background thread polls a client for
utilisation metrics every ``check_interval_in_sec`` and ``is_host_idle()`` tells the watchdog
whether the accelerators of this host are idle (a hang) or busy (a slow step).
"""

from __future__ import annotations

import threading
from typing import Optional

from axlearn_b200.common.config import REQUIRED, Configurable, InstantiableConfig, Required, config_class


class DeviceMonitorClient(Configurable):
    """Source of utilisation numbers; the base class reports "never idle"."""

    @config_class
    class Config(Configurable.Config):
        pass

    def collect_metrics(self) -> list[dict]:
        """One dict per device with at least ``util`` (percent) and ``mem_used_frac``."""
        return []

    def is_host_idle(self, metrics: list[dict]) -> bool:
        del metrics
        return False


class DeviceMonitor(Configurable):
    @config_class
    class Config(Configurable.Config):
        monitor_client: InstantiableConfig = DeviceMonitorClient.default_config()
        check_interval_in_sec: float = 60.0
        log_every_n: int = 1

    def __init__(self, cfg):
        super().__init__(cfg)
        self._client = cfg.monitor_client.instantiate()
        self._idle = False
        self._last: list[dict] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()
        self._checks = 0

    def _check_once(self) -> None:
        metrics = self._client.collect_metrics()
        idle = self._client.is_host_idle(metrics)
        with self._lock:
            self._last, self._idle = metrics, idle
            self._checks += 1

    def _loop(self) -> None:
        while not self._stop.wait(self._config.check_interval_in_sec):
            try:
                self._check_once()
            except Exception as e:  # pylint: disable=broad-except
                print(f"[device monitor] metric collection failed: {e!r}", flush=True)

    def start_monitoring(self) -> None:
        if self._config.check_interval_in_sec <= 0 or self._thread is not None:
            return
        self._stop.clear()
        self._check_once()
        self._thread = threading.Thread(target=self._loop, name="device-monitor", daemon=True)
        self._thread.start()

    def stop_monitoring(self) -> None:
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=5)
            self._thread = None

    def is_host_idle(self) -> bool:
        with self._lock:
            return self._idle

    def last_metrics(self) -> list[dict]:
        with self._lock:
            return list(self._last)
