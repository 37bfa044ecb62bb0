"""Fault-tolerance agent: supervises one trainer process, detects crashes and hangs, restarts it.

Parity targets in the reference (axlearn/ft/agent.py:106-251, axlearn/ft/monitor.py:42-225,
README): the pod's main process is the agent; it spawns the trainer, follows its output to learn
the current step, declares a hang when the step has not advanced for ``hang_timeout_seconds``,
restarts the trainer on crash / hang (the trainer resumes from the latest checkpoint by
itself), counts restarts, gives up after ``max_restarts`` (the reference then falls back to a
pod restart), and reports its state to a manager that coordinates restarts across workers
(``axlearn_b200/ft/manager.py``).

Everything here is host-side: a trainer is a child process, a failure is an exit code, a missed
heartbeat or a step counter that stopped moving.  Nothing ever makes a GPU fault or hang to test
this; GPU-side waits are bounded and report through a status word instead
(``axlearn_b200/ops/cuda_ops.py: check_status``).
"""

from __future__ import annotations

import dataclasses
import enum
import os
import re
import signal
import subprocess
import sys
import threading
import time
from typing import Callable, Optional, Sequence

STEP_PATTERN = re.compile(r"(?:^|\s)step[ =:]+(\d+)")


class WorkerState(enum.Enum):
    STARTING = "starting"
    RUNNING = "running"
    HUNG = "hung"
    CRASHED = "crashed"
    RESTARTING = "restarting"   # stopped on the manager's request (another worker failed)
    FINISHED = "finished"
    FAILED = "failed"     # gave up after max_restarts


@dataclasses.dataclass
class AgentReport:
    state: WorkerState
    step: int
    restarts: int
    last_exit_code: Optional[int]
    reason: str = ""


class TrainerProcess:
    """One run of the trainer command, with its output followed on a thread."""

    def __init__(self, command: Sequence[str], *, env: Optional[dict] = None, log_path: Optional[str] = None,
                 on_line: Optional[Callable[[str], None]] = None):
        self._log = open(log_path, "a", encoding="utf-8") if log_path else None  # pylint: disable=consider-using-with
        # A supervised trainer may be killed at any moment (kill() below).  A rank that dies while
        # its memory is bound to an NVLink multicast object raises NVLink faults on its peers'
        # GPUs, so supervised runs keep NCCL's in-switch reduction and symmetric-memory multicast
        # off unless the caller's environment says otherwise.
        env = dict(os.environ if env is None else env)
        env.setdefault("NCCL_NVLS_ENABLE", "0")
        env.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.proc = subprocess.Popen(  # pylint: disable=consider-using-with
            list(command), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env,
            start_new_session=True)
        self.step = -1
        self.last_progress = time.time()
        self._on_line = on_line
        self._reader = threading.Thread(target=self._follow, name="trainer-output", daemon=True)
        self._reader.start()

    def _follow(self) -> None:
        assert self.proc.stdout is not None
        for line in self.proc.stdout:
            if self._log is not None:
                self._log.write(line)
                self._log.flush()
            m = STEP_PATTERN.search(line)
            if m:
                step = int(m.group(1))
                if step != self.step:
                    self.step, self.last_progress = step, time.time()
            if self._on_line is not None:
                self._on_line(line)

    def poll(self) -> Optional[int]:
        return self.proc.poll()

    def kill(self) -> None:
        """Ends exactly this trainer's process group."""
        if self.proc.poll() is None:
            try:
                os.killpg(self.proc.pid, signal.SIGKILL)
            except ProcessLookupError:
                pass
        self.proc.wait()
        self._reader.join(timeout=5)
        if self._log is not None:
            self._log.close()


class Agent:
    def __init__(self, command: Sequence[str], *, hang_timeout_seconds: float = 600.0,
                 startup_timeout_seconds: Optional[float] = None, max_restarts: int = 3,
                 poll_interval_seconds: float = 0.2, env: Optional[dict] = None, log_path: Optional[str] = None,
                 report_fn: Optional[Callable[[AgentReport], Optional[str]]] = None):
        self._command = list(command)
        self._hang_timeout = hang_timeout_seconds
        self._startup_timeout = startup_timeout_seconds or hang_timeout_seconds
        self._max_restarts = max_restarts
        self._poll = poll_interval_seconds
        self._env = env
        self._log_path = log_path
        # report_fn sends a report (e.g. to the manager) and may return a command: "restart".
        self._report_fn = report_fn
        self.restarts = 0
        self.history: list[AgentReport] = []
        self._last_step = -1

    def _report(self, state: WorkerState, trainer: Optional[TrainerProcess], code: Optional[int], reason="") -> Optional[str]:
        step = trainer.step if trainer is not None and trainer.step >= 0 else self._last_step
        rep = AgentReport(state=state, step=step, restarts=self.restarts, last_exit_code=code, reason=reason)
        self.history.append(rep)
        return self._report_fn(rep) if self._report_fn is not None else None

    def run(self) -> AgentReport:
        """Supervises until the trainer exits 0 (FINISHED) or restarts are exhausted (FAILED)."""
        while True:
            trainer = TrainerProcess(self._command, env=self._env, log_path=self._log_path)
            self._report(WorkerState.STARTING, trainer, None)
            outcome, code, reason = self._supervise(trainer)
            self._last_step = max(self._last_step, trainer.step)
            trainer.kill()
            if outcome == WorkerState.FINISHED:
                self._report(WorkerState.FINISHED, trainer, code)
                return self.history[-1]
            self._report(outcome, trainer, code, reason)
            if self.restarts >= self._max_restarts:
                self._report(WorkerState.FAILED, trainer, code, f"gave up after {self.restarts} restarts")
                return self.history[-1]
            self.restarts += 1

    def _supervise(self, trainer: TrainerProcess):
        announced_running = False
        while True:
            code = trainer.poll()
            if code is not None:
                time.sleep(0.05)  # let the reader drain the last lines
                return (WorkerState.FINISHED, code, "") if code == 0 else (WorkerState.CRASHED, code, f"exit code {code}")
            stalled = time.time() - trainer.last_progress
            limit = self._hang_timeout if trainer.step >= 0 else self._startup_timeout
            if stalled > limit:
                return WorkerState.HUNG, None, f"step {trainer.step} unchanged for {stalled:.1f}s"
            if trainer.step >= 0:
                cmd = self._report(WorkerState.RUNNING, trainer, None) if (not announced_running or self._report_fn) else None
                announced_running = True
                if cmd == "restart":
                    return WorkerState.RESTARTING, None, "restart requested by the manager"
            time.sleep(self._poll)


def main(argv: Optional[Sequence[str]] = None) -> int:
    """``python -m axlearn_b200.ft.agent [--hang-timeout S] [--max-restarts N] -- <trainer command...>``"""
    import argparse

    argv = list(sys.argv[1:] if argv is None else argv)
    if "--" not in argv:
        print("usage: agent [options] -- <trainer command>", file=sys.stderr)
        return 2
    split = argv.index("--")
    ap = argparse.ArgumentParser()
    ap.add_argument("--hang-timeout", type=float, default=600.0)
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--log", default=None)
    ap.add_argument("--manager", default=None, help="host:port of the ft manager")
    ap.add_argument("--worker-id", default=os.environ.get("RANK", "0"))
    args = ap.parse_args(argv[:split])
    report_fn = None
    if args.manager:
        from axlearn_b200.ft.manager import ManagerClient

        host, port = args.manager.rsplit(":", 1)
        client = ManagerClient(host, int(port), worker_id=args.worker_id)
        report_fn = client.report
    agent = Agent(argv[split + 1:], hang_timeout_seconds=args.hang_timeout, max_restarts=args.max_restarts,
                  log_path=args.log, report_fn=report_fn)
    final = agent.run()
    print(f"[ft agent] {final.state.value} at step {final.step} after {final.restarts} restarts", flush=True)
    return 0 if final.state == WorkerState.FINISHED else 1


if __name__ == "__main__":
    sys.exit(main())
