"""Coordination of fault-tolerance agents: when one worker's trainer dies, all restart together.

Parity targets in the reference (axlearn/ft/manager.proto:117-133, manager_server.py:40-700,
manager_client.py): workers report to a replica manager, replica managers to a global manager;
a failure anywhere bumps a *restart generation* and every worker restarts its trainer so that
the collective job resumes from the same checkpoint.  Stragglers are flagged from reported step
rates (the reference uses tensor-core utilisation, axlearn/ft/monitor.py:42-225).

Transport: newline-delimited JSON over TCP (the reference uses gRPC with generated stubs; the
protocol here is three message types -- report, command, status -- and needs no code
generation).  A ``Manager`` with ``upstream=(host, port)`` forwards failures to, and receives
generations from, a higher-level manager, which gives the same worker -> replica -> global
hierarchy.
"""

from __future__ import annotations

import json
import socket
import socketserver
import threading
import time
from typing import Optional


class _Handler(socketserver.StreamRequestHandler):
    def handle(self):
        manager: "Manager" = self.server.manager  # type: ignore[attr-defined]
        for raw in self.rfile:
            try:
                msg = json.loads(raw)
            except json.JSONDecodeError:
                continue
            reply = manager.handle(msg)
            self.wfile.write((json.dumps(reply) + "\n").encode())
            self.wfile.flush()


class _Server(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True


class Manager:
    """Tracks workers, turns any failure into a job-wide restart generation."""

    def __init__(self, host: str = "127.0.0.1", port: int = 0, *, heartbeat_timeout_seconds: float = 30.0,
                 straggler_ratio: float = 0.5, upstream: Optional[tuple] = None, manager_id: str = "manager"):
        self._lock = threading.Lock()
        self.generation = 0
        self.workers: dict[str, dict] = {}
        self._heartbeat_timeout = heartbeat_timeout_seconds
        self._straggler_ratio = straggler_ratio
        self._server = _Server((host, port), _Handler)
        self._server.manager = self  # type: ignore[attr-defined]
        self._thread = threading.Thread(target=self._server.serve_forever, name="ft-manager", daemon=True)
        self._upstream = ManagerClient(*upstream, worker_id=manager_id) if upstream else None
        self.events: list[tuple] = []

    @property
    def address(self) -> tuple:
        return self._server.server_address

    def start(self) -> "Manager":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._server.shutdown()
        self._server.server_close()

    # ------------------------------------------------------------------ protocol
    def handle(self, msg: dict) -> dict:
        kind = msg.get("type")
        if kind == "report":
            return self._on_report(msg)
        if kind == "status":
            return self.status()
        return {"error": f"unknown message type {kind!r}"}

    def _bump(self, why: str) -> None:
        self.generation += 1
        self.events.append((time.time(), self.generation, why))

    def _on_report(self, msg: dict) -> dict:
        wid = str(msg["worker_id"])
        now = time.time()
        with self._lock:
            w = self.workers.setdefault(wid, {"generation": self.generation, "step": -1, "state": "starting",
                                              "first_step_time": None, "first_step": None})
            prev_state = w["state"]
            w.update(state=msg["state"], restarts=msg.get("restarts", 0), last_seen=now)
            step = int(msg.get("step", -1))
            if step >= 0 and step != w["step"]:
                if w["first_step"] is None:
                    w["first_step"], w["first_step_time"] = step, now
                w["step"], w["step_time"] = step, now
            failed = msg["state"] in ("crashed", "hung") and prev_state not in ("crashed", "hung")
            if failed and w["generation"] == self.generation:
                # First news of this failure: everyone restarts.
                self._bump(f"worker {wid} {msg['state']}: {msg.get('reason', '')}")
                if self._upstream is not None:
                    up = self._upstream.send({"type": "report", "worker_id": self._upstream.worker_id,
                                              "state": msg["state"], "step": step, "reason": msg.get("reason", "")})
                    self.generation = max(self.generation, int(up.get("generation", 0)))
            if msg["state"] in ("starting",):
                w["generation"] = self.generation
            command = None
            if msg["state"] == "running" and w["generation"] < self.generation:
                command = "restart"
                w["generation"] = self.generation
            return {"generation": self.generation, "command": command}

    def poll_upstream(self) -> None:
        """Pulls the generation from the higher-level manager (called periodically by owners)."""
        if self._upstream is None:
            return
        up = self._upstream.send({"type": "status"})
        with self._lock:
            if int(up.get("generation", 0)) > self.generation:
                self.generation = int(up["generation"])
                self.events.append((time.time(), self.generation, "generation from upstream"))

    def status(self) -> dict:
        now = time.time()
        with self._lock:
            workers = {}
            rates = {}
            for wid, w in self.workers.items():
                alive = now - w.get("last_seen", 0) <= self._heartbeat_timeout
                workers[wid] = {"state": w["state"], "step": w["step"], "alive": alive,
                                "restarts": w.get("restarts", 0)}
                if w.get("first_step") is not None and w["step"] > w["first_step"]:
                    rates[wid] = (w["step"] - w["first_step"]) / max(1e-6, w["step_time"] - w["first_step_time"])
            stragglers = []
            if len(rates) >= 2:
                best = max(rates.values())
                stragglers = sorted(w for w, r in rates.items() if r < self._straggler_ratio * best)
            missing = sorted(w for w, v in workers.items() if not v["alive"] and v["state"] not in ("finished", "failed"))
            return {"generation": self.generation, "workers": workers, "stragglers": stragglers,
                    "missing_heartbeats": missing}


class ManagerClient:
    """One TCP connection per call keeps the client trivially robust to manager restarts."""

    def __init__(self, host: str, port: int, *, worker_id: str, timeout_seconds: float = 5.0,
                 drop_fn=None):
        self._addr = (host, port)
        self.worker_id = worker_id
        self._timeout = timeout_seconds
        # Test hook: drop_fn(msg) -> True simulates a lost message.
        self._drop_fn = drop_fn

    def send(self, msg: dict) -> dict:
        if self._drop_fn is not None and self._drop_fn(msg):
            return {}
        try:
            with socket.create_connection(self._addr, timeout=self._timeout) as s:
                s.sendall((json.dumps(msg) + "\n").encode())
                s.shutdown(socket.SHUT_WR)
                data = b""
                while not data.endswith(b"\n"):
                    chunk = s.recv(65536)
                    if not chunk:
                        break
                    data += chunk
            return json.loads(data) if data else {}
        except (OSError, json.JSONDecodeError):
            return {}

    def report(self, rep) -> Optional[str]:
        """``Agent(report_fn=client.report)``: forwards an AgentReport, returns the manager's command."""
        reply = self.send({"type": "report", "worker_id": self.worker_id, "state": rep.state.value, "step": rep.step,
                           "restarts": rep.restarts, "reason": rep.reason})
        return reply.get("command")
