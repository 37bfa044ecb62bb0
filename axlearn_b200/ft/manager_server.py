"""The worker -> replica manager -> global manager hierarchy of the fault-tolerance service.

Parity target: the reference's ``ManagerServer`` and its six RPCs (axlearn/ft/manager.proto:
117-133; axlearn/ft/manager_server.py:40-700):

==========================  ==========================================  =========================
reference RPC               direction                                   message ``type`` here
==========================  ==========================================  =========================
``ReportStatus``            worker -> its replica manager               ``report_status``
``ReportReplicaStatus``     replica manager -> global manager           ``report_replica_status``
``RestartReplicaTraining``  global manager -> replica manager           ``restart_replica``
``RestartTraining``         replica manager -> worker                   (reply to ``report_status``)
``ReportPodShutdown``       worker -> replica manager (-> global)       ``report_pod_shutdown``
``RequestGlobalRestart``    any worker -> global manager                ``request_global_restart``
==========================  ==========================================  =========================

A *replica* is one data-parallel copy of the job (one slice / node group).  The first worker of
each replica runs a ``ReplicaManager``; the first replica's host also runs the ``GlobalManager``.
Workers report step, state and device utilisation to their replica manager, which aggregates
and forwards a ``ReplicaStatus``; the global manager keeps the detailed view that the monitors
(``axlearn_b200.ft.monitor``) read.

Restarts are *counted*: the global manager owns ``global_restart_count``; a restart request
carries the requester's count and is ignored when that count is stale (several workers of a
dying job all ask at once: only the first one starts a new generation).  ``restart_replica``
tells a replica manager the new count; its workers learn it from the reply to their next
status report (there is no connection from the manager back into a worker, so the reference's
``RestartTraining`` push becomes a pull) and restart their trainers.

Transport is the newline-delimited JSON over TCP of ``axlearn_b200.ft.manager``: no generated
stubs, every call is one short-lived connection.
"""

from __future__ import annotations

import threading
import time
from typing import Optional

from axlearn_b200.ft.manager import ManagerClient, _Handler, _Server

ROLE_REPLICA, ROLE_GLOBAL = "replica", "global"
UTIL_UNAVAILABLE = -1.0


class _Base:
    def __init__(self, host: str, port: int, name: str):
        self._lock = threading.Lock()
        self._server = _Server((host, port), _Handler)
        self._server.manager = self  # type: ignore[attr-defined]
        self._thread = threading.Thread(target=self._server.serve_forever, name=name, daemon=True)
        self.events: list[tuple] = []

    @property
    def address(self) -> tuple:
        return self._server.server_address

    def start(self):
        self._thread.start()
        return self

    def stop(self) -> None:
        self._server.shutdown()
        self._server.server_close()

    def _log(self, what: str) -> None:
        self.events.append((time.time(), what))


class GlobalManager(_Base):
    """Top of the hierarchy: the detailed job view and the restart counter."""

    role = ROLE_GLOBAL

    def __init__(self, host: str = "127.0.0.1", port: int = 0, *, num_replicas: int = 1):
        super().__init__(host, port, "ft-global-manager")
        self.num_replicas = num_replicas
        self.global_restart_count = 0
        self.replicas: dict[int, dict] = {}
        self.shutdowns: list[dict] = []

    # ------------------------------------------------------------------ protocol
    def handle(self, msg: dict) -> dict:
        kind = msg.get("type")
        if kind == "report_replica_status":
            return self._on_replica_status(msg)
        if kind == "request_global_restart":
            return self.request_global_restart(msg.get("worker_identity", {}), msg.get("reason", ""),
                                               int(msg.get("restart_count", 0)))
        if kind == "report_pod_shutdown":
            return self._on_pod_shutdown(msg)
        if kind == "status":
            return self.get_detailed_global_status()
        return {"error": f"global manager: unknown message type {kind!r}"}

    def _on_replica_status(self, msg: dict) -> dict:
        rid = int(msg["replica_id"])
        with self._lock:
            self.replicas[rid] = {"workers": msg.get("workers", []), "address": msg.get("address"),
                                  "restart_count": int(msg.get("restart_count", 0)), "last_update": time.time()}
            return {"acknowledged": True, "global_restart_count": self.global_restart_count}

    def request_global_restart(self, identity: dict, reason: str, restart_count: int) -> dict:
        """Starts a new generation unless the requester is behind one that already started."""
        with self._lock:
            if restart_count < self.global_restart_count:
                return {"acknowledged": False, "message": "stale restart count",
                        "global_restart_count": self.global_restart_count}
            self.global_restart_count += 1
            count = self.global_restart_count
            targets = {rid: r.get("address") for rid, r in self.replicas.items()}
            self._log(f"global restart {count}: {reason} (asked by {identity})")
        results = self._restart_all_replicas(targets, reason, count)
        return {"acknowledged": True, "message": f"restart {count}", "global_restart_count": count,
                "replicas_acknowledged": results}

    def _restart_all_replicas(self, targets: dict, reason: str, count: int) -> dict:
        out = {}
        for rid, addr in targets.items():
            if not addr:
                out[str(rid)] = False
                continue
            reply = ManagerClient(addr[0], int(addr[1]), worker_id="global").send(
                {"type": "restart_replica", "reason": reason, "restart_count": count})
            out[str(rid)] = bool(reply.get("acknowledged"))
        return out

    def send_restart_to_all_replicas(self, reason: str) -> dict:
        """What the hang monitor calls: a restart request from the global manager itself."""
        with self._lock:
            count = self.global_restart_count
        return self.request_global_restart({"hostname": "global-manager"}, reason, count).get(
            "replicas_acknowledged", {})

    def _on_pod_shutdown(self, msg: dict) -> dict:
        with self._lock:
            self.shutdowns.append({"worker_identity": msg.get("worker_identity", {}), "reason": msg.get("reason", ""),
                                   "time": time.time()})
            count = self.global_restart_count
        # A pod that goes away takes its replica's collective down with it: restart everyone.
        return self.request_global_restart(msg.get("worker_identity", {}), f"pod shutdown: {msg.get('reason', '')}",
                                           count)

    # ------------------------------------------------------------------ views
    def get_global_status(self) -> dict:
        with self._lock:
            workers = sum(len(r["workers"]) for r in self.replicas.values())
            return {"replicas": len(self.replicas), "expected_replicas": self.num_replicas, "workers": workers,
                    "global_restart_count": self.global_restart_count}

    def get_detailed_global_status(self) -> dict:
        with self._lock:
            return {"global_restart_count": self.global_restart_count,
                    "replicas": {rid: {"workers": [dict(w) for w in r["workers"]], "restart_count": r["restart_count"],
                                       "last_update": r["last_update"]} for rid, r in self.replicas.items()}}


class ReplicaManager(_Base):
    """Middle tier: the workers of one replica report here; failures go up, restarts come down."""

    role = ROLE_REPLICA

    def __init__(self, replica_id: int, host: str = "127.0.0.1", port: int = 0, *,
                 global_address: Optional[tuple] = None):
        super().__init__(host, port, f"ft-replica-manager-{replica_id}")
        self.replica_id = replica_id
        self.restart_count = 0
        self.workers: dict[int, dict] = {}
        self._global = ManagerClient(global_address[0], int(global_address[1]), worker_id=f"replica-{replica_id}") \
            if global_address else None

    def handle(self, msg: dict) -> dict:
        kind = msg.get("type")
        if kind == "report_status":
            return self._on_worker_status(msg)
        if kind == "restart_replica":
            return self._on_restart_replica(msg)
        if kind == "report_pod_shutdown":
            return self._forward(msg)
        if kind == "request_global_restart":
            return self._forward(msg)
        if kind == "status":
            return self.get_replica_status()
        return {"error": f"replica manager: unknown message type {kind!r}"}

    def _forward(self, msg: dict) -> dict:
        if self._global is None:
            return {"acknowledged": False, "message": "no global manager configured"}
        return self._global.send(msg) or {"acknowledged": False, "message": "global manager unreachable"}

    def _on_worker_status(self, msg: dict) -> dict:
        ident = msg.get("worker_identity", {})
        wid = int(ident.get("worker_id", 0))
        now = time.time()
        with self._lock:
            w = self.workers.setdefault(wid, {"worker_identity": ident, "step": -1, "last_update": now})
            step = int(msg.get("step", -1))
            if step != w["step"]:
                w["step"], w["last_update"] = step, now  # progress, not mere liveness
            w.update(worker_identity=ident, state=msg.get("state", "running"), last_seen=now,
                     restart_count=int(msg.get("restart_count", 0)),
                     tensorcore_util=float(msg.get("tensorcore_util", UTIL_UNAVAILABLE)))
            behind = w["restart_count"] < self.restart_count
            reply = {"acknowledged": True, "restart_count": self.restart_count,
                     "command": "restart" if behind and msg.get("state") == "running" else None}
            failed = msg.get("state") in ("crashed", "hung")
            count = w["restart_count"]
        if failed:
            up = self._forward({"type": "request_global_restart", "worker_identity": ident,
                                "reason": f"worker {wid} of replica {self.replica_id} {msg.get('state')}: "
                                          f"{msg.get('reason', '')}", "restart_count": count})
            reply["global"] = up
        return reply

    def _on_restart_replica(self, msg: dict) -> dict:
        with self._lock:
            self.restart_count = max(self.restart_count, int(msg.get("restart_count", self.restart_count + 1)))
            self._log(f"restart {self.restart_count}: {msg.get('reason', '')}")
            return {"acknowledged": True, "restart_count": self.restart_count, "workers": len(self.workers)}

    def get_replica_status(self) -> dict:
        with self._lock:
            return {"replica_id": self.replica_id, "restart_count": self.restart_count, "address": list(self.address),
                    "workers": [dict(w) for _, w in sorted(self.workers.items())]}

    def report_replica_status(self) -> dict:
        """Pushes the aggregated view up (the replica manager's monitor loop calls this)."""
        if self._global is None:
            return {}
        status = self.get_replica_status()
        reply = self._global.send({"type": "report_replica_status", **status})
        with self._lock:
            self.restart_count = max(self.restart_count, int(reply.get("global_restart_count", 0)))
        return reply


class WorkerClient:
    """What an agent uses to talk to its replica manager."""

    def __init__(self, address: tuple, *, replica_id: int, worker_id: int, hostname: str = "localhost", drop_fn=None):
        self._client = ManagerClient(address[0], int(address[1]), worker_id=f"{replica_id}/{worker_id}", drop_fn=drop_fn)
        self.identity = {"replica_id": replica_id, "worker_id": worker_id, "hostname": hostname}
        self.restart_count = 0

    def report_status(self, *, step: int, state: str = "running", tensorcore_util: float = UTIL_UNAVAILABLE,
                      reason: str = "") -> Optional[str]:
        reply = self._client.send({"type": "report_status", "worker_identity": self.identity, "step": step,
                                   "state": state, "restart_count": self.restart_count, "reason": reason,
                                   "tensorcore_util": tensorcore_util})
        if reply.get("command") == "restart":
            self.restart_count = int(reply["restart_count"])
            return "restart"
        return None

    def report(self, rep) -> Optional[str]:
        """``Agent(report_fn=client.report)``."""
        if rep.state.value == "starting":
            # A trainer that (re)starts has caught up with whatever generation was announced.
            reply = self._client.send({"type": "status"})
            self.restart_count = max(self.restart_count, int(reply.get("restart_count", 0)))
        return self.report_status(step=rep.step, state=rep.state.value, reason=rep.reason)

    def report_pod_shutdown(self, reason: str) -> dict:
        return self._client.send({"type": "report_pod_shutdown", "worker_identity": self.identity, "reason": reason})

    def request_global_restart(self, reason: str) -> dict:
        return self._client.send({"type": "request_global_restart", "worker_identity": self.identity, "reason": reason,
                                  "restart_count": self.restart_count})
