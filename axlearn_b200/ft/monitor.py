"""Straggler and hang monitors of the fault-tolerance service.

Parity targets: ``StragglerMonitor`` (axlearn/ft/monitor.py:42-225) and the hang / restart part
of ``StatusMonitor`` (:227-600).

``StragglerMonitor`` reads the global manager's detailed status (per replica, per worker: the
utilisation figure the worker reported) and flags workers whose utilisation deviates from the
job's median by more than ``sensitivity`` robust standard deviations (median absolute deviation
scaled by 0.6745).  A worker is only *reported* after it has been an outlier continuously:
"potential" after half of ``sustained_duration_seconds``, "confirmed" after all of it.  The
reference feeds it TPU tensor-core utilisation; here workers report the GPU utilisation that
``axlearn_b200.common.monitoring.gpu_client`` reads from NVML (read-only), or any figure with
"busier is larger" meaning, e.g. steps per second.

``StatusMonitor`` runs beside a manager: a replica is *hanging* when none of its workers has
advanced its step for ``hang_threshold_seconds``; any hanging replica makes the global manager
restart all replicas (a collective job cannot continue with a part of it stalled).

Nothing here touches a GPU: both monitors work on numbers that workers report, and their tests
drive them with fabricated reports.
"""

from __future__ import annotations

import statistics
import threading
import time
from typing import Callable, Optional

STRAGGLER_POTENTIAL = "POTENTIAL STRAGGLER"
STRAGGLER_CONFIRMED = "CONFIRMED STRAGGLER"


class StragglerMonitor:
    _CONSISTENCY_CONSTANT = 0.6745  # MAD -> standard-deviation units for normal data

    def __init__(self, *, enabled: bool = True, sensitivity: float = 8.0, sustained_duration_seconds: float = 300.0,
                 min_workers: int = 4, now_fn: Callable[[], float] = time.time,
                 log_fn: Optional[Callable[[str], None]] = None):
        self.enabled = enabled
        self.sensitivity = sensitivity
        self.sustained_duration_seconds = sustained_duration_seconds
        self.min_workers = min_workers
        self._now = now_fn
        self._log = log_fn or (lambda s: print(s, flush=True))
        self._since: dict[tuple[int, int], float] = {}
        self.reports: list[dict] = []

    def reset(self) -> None:
        self._since.clear()

    def run_check(self, detailed_status: dict) -> list[dict]:
        """One pass over a ``GlobalManager.get_detailed_global_status()`` dict; returns (and logs)
        the workers that crossed a reporting threshold in this pass."""
        if not self.enabled:
            return []
        workers = []
        for rid, info in detailed_status.get("replicas", {}).items():
            for w in info.get("workers", []):
                util = float(w.get("tensorcore_util", -1.0))
                if util < 0:
                    continue
                ident = w.get("worker_identity", {})
                workers.append((int(rid), int(ident.get("worker_id", -1)), ident.get("hostname", "unknown"), util))
        if len(workers) < self.min_workers:
            return []
        values = [w[3] for w in workers]
        median = statistics.median(values)
        mad = statistics.median(abs(v - median) for v in values)
        if mad == 0:
            self._since.clear()  # all alike: no outlier is possible
            return []
        now = self._now()
        current = set()
        out = []
        for rid, wid, host, util in workers:
            z = self._CONSISTENCY_CONSTANT * (util - median) / mad
            if abs(z) < self.sensitivity:
                continue
            key = (rid, wid)
            current.add(key)
            since = self._since.setdefault(key, now)
            duration = now - since
            label = None
            if duration >= self.sustained_duration_seconds:
                label = STRAGGLER_CONFIRMED
            elif duration >= self.sustained_duration_seconds / 2:
                label = STRAGGLER_POTENTIAL
            if label is not None:
                rep = {"label": label, "replica_id": rid, "worker_id": wid, "hostname": host, "util": util,
                       "median": median, "mean": statistics.mean(values), "modified_z": z, "duration": duration}
                out.append(rep)
                self._log(f"FT monitor: {label} - replica {rid} worker {wid} ({host}): utilisation {util:.1f} vs "
                          f"job median {median:.1f}; outlier for {int(duration)} s (modified z {z:.1f}, "
                          f"sensitivity {self.sensitivity:.1f})")
        for key in list(self._since):
            if key not in current:
                del self._since[key]
        self.reports.extend(out)
        return out


class StatusMonitor:
    """Periodic duties of a manager process: replica managers push their status up; the global
    manager looks for hanging replicas and stragglers."""

    def __init__(self, *, global_manager=None, replica_manager=None, hang_threshold_seconds: float = 600.0,
                 interval_seconds: float = 10.0, straggler_monitor: Optional[StragglerMonitor] = None,
                 now_fn: Callable[[], float] = time.time):
        self._global = global_manager
        self._replica = replica_manager
        self.hang_threshold_seconds = hang_threshold_seconds
        self._interval = interval_seconds
        self._straggler = straggler_monitor
        self._now = now_fn
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.restarts_triggered: list[str] = []

    @property
    def is_global_manager(self) -> bool:
        return self._global is not None

    @property
    def is_replica_manager(self) -> bool:
        return self._replica is not None

    def count_hanging_replicas(self, replicas: dict) -> int:
        now = self._now()
        hanging = 0
        for info in replicas.values():
            workers = info.get("workers", [])
            if workers and all(now - w.get("last_update", 0) >= self.hang_threshold_seconds for w in workers):
                hanging += 1
        return hanging

    def detect_global_training_hang(self) -> bool:
        if not self.is_global_manager:
            return False
        replicas = self._global.get_detailed_global_status().get("replicas", {})
        return bool(replicas) and self.count_hanging_replicas(replicas) > 0

    def trigger_global_restart(self, reason: str) -> bool:
        if not self.is_global_manager:
            return False
        results = self._global.send_restart_to_all_replicas(reason)
        self.restarts_triggered.append(reason)
        return any(results.values())

    def run_once(self) -> None:
        if self.is_replica_manager:
            self._replica.report_replica_status()
        if self.is_global_manager:
            if self.detect_global_training_hang():
                self.trigger_global_restart(f"no progress for {self.hang_threshold_seconds} s in a replica")
            if self._straggler is not None:
                self._straggler.run_check(self._global.get_detailed_global_status())

    def start(self) -> "StatusMonitor":
        def loop():
            while not self._stop.wait(self._interval):
                try:
                    self.run_once()
                except Exception as e:  # pylint: disable=broad-except
                    print(f"FT monitor: {type(e).__name__}: {e}", flush=True)

        self._thread = threading.Thread(target=loop, name="ft-status-monitor", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
