"""NVML-backed device monitor client (read-only queries).

Parity targets in the reference: ``GPUMonitorClient`` (axlearn/common/monitoring/gpu_client.py)
and ``gpu_device_monitor.py``.  Only *reads* NVML (utilisation, memory, clocks, throttle
reasons); nothing here changes a GPU setting.  ``nvml`` can be injected as a factory (tests use a fake with
the same calls), otherwise ``pynvml`` is imported lazily.
"""

from __future__ import annotations

from typing import Any, Optional

from axlearn_b200.common.config import config_class
from axlearn_b200.common.monitoring.device_monitor import DeviceMonitorClient


class GPUMonitorClient(DeviceMonitorClient):
    @config_class
    class Config(DeviceMonitorClient.Config):
        # A host counts as idle when every GPU is below this SM utilisation (percent).
        idle_util_threshold: float = 5.0
        # Zero-argument callable returning the NVML module (or a stand-in with the same calls);
        # None = import pynvml.
        nvml: Optional[Any] = None

    def __init__(self, cfg):
        super().__init__(cfg)
        self._nvml = cfg.nvml() if cfg.nvml is not None else None
        self._ready = False

    def _lib(self):
        if self._nvml is None:
            import pynvml  # pylint: disable=import-outside-toplevel

            self._nvml = pynvml
        if not self._ready:
            self._nvml.nvmlInit()
            self._ready = True
        return self._nvml

    def collect_metrics(self) -> list[dict]:
        n = self._lib()
        out = []
        for i in range(n.nvmlDeviceGetCount()):
            h = n.nvmlDeviceGetHandleByIndex(i)
            util = n.nvmlDeviceGetUtilizationRates(h)
            mem = n.nvmlDeviceGetMemoryInfo(h)
            out.append({"index": i, "util": float(util.gpu), "mem_util": float(util.memory),
                        "mem_used_frac": float(mem.used) / max(1.0, float(mem.total))})
        return out

    def is_host_idle(self, metrics: list[dict]) -> bool:
        return bool(metrics) and all(m["util"] < self._config.idle_util_threshold for m in metrics)
