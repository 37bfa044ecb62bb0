"""Failure detection and recovery, with every failure injected on the host.

Trainers are CPU child processes; a failure is an exception, a process that stops making
progress, or a dropped message.  No GPU is involved and nothing is ever made to fault or hang a
device (GPU-side waits are bounded and report through a status word; see test_gpu_fused_comm).
"""

import os
import subprocess
import sys
import threading
import time
import types
import urllib.request

import pytest
import torch

from axlearn_b200.common.liveness_monitor import LivenessMonitor
from axlearn_b200.common.monitoring.device_monitor import DeviceMonitor
from axlearn_b200.common.monitoring.gpu_client import GPUMonitorClient
from axlearn_b200.common.status_server import StatusHTTPServer
from axlearn_b200.ft.agent import Agent, WorkerState
from axlearn_b200.ft.manager import Manager, ManagerClient

HERE = os.path.dirname(os.path.abspath(__file__))
SCRIPT = os.path.join(HERE, "ft_trainer_script.py")


def _trainer_cmd(trainer_dir, max_step=8):
    return [sys.executable, SCRIPT, "--module=text.gpt.c4_trainer", "--config=fuji-test-v1",
            f"--trainer_dir={trainer_dir}", f"--max_step={max_step}", "--save_every_n_steps=2",
            "--log_every_n_steps=1", "--device=cpu"]


def _final_state(trainer_dir):
    from axlearn_b200.common.checkpointer import latest_checkpoint_path, read_state_tensors

    path = latest_checkpoint_path(os.path.join(trainer_dir, "checkpoints"))
    return path, read_state_tensors(path)


@pytest.fixture(scope="module")
def uninterrupted(tmp_path_factory):
    d = tmp_path_factory.mktemp("clean")
    subprocess.run(_trainer_cmd(d), check=True, capture_output=True, timeout=300)
    return _final_state(str(d))


@pytest.mark.parametrize("kind", ["crash", "hang"])
def test_agent_restarts_trainer_and_resume_is_bit_exact(tmp_path, uninterrupted, kind):
    env = dict(os.environ, AXB_FAULT=f"{kind}@5", AXB_FAULT_MARKER=str(tmp_path / "fault_fired"))
    agent = Agent(_trainer_cmd(tmp_path / "run"), hang_timeout_seconds=6.0, startup_timeout_seconds=120.0,
                  max_restarts=2, env=env, log_path=str(tmp_path / "trainer.log"))
    final = agent.run()
    assert final.state == WorkerState.FINISHED and final.restarts == 1, agent.history
    states = [h.state for h in agent.history]
    assert (WorkerState.CRASHED if kind == "crash" else WorkerState.HUNG) in states
    log = open(tmp_path / "trainer.log", encoding="utf-8").read()
    # The second run resumed from the checkpoint at step 4 instead of starting over.
    assert log.count("[trainer] step 1 ") == 1 and log.count("[trainer] step 8 ") == 1
    ref_path, ref = uninterrupted
    path, got = _final_state(str(tmp_path / "run"))
    assert os.path.basename(path) == os.path.basename(ref_path)
    assert set(got) == set(ref)
    for k in ref:
        assert torch.equal(got[k], ref[k]), k


def test_agent_gives_up_after_max_restarts(tmp_path):
    agent = Agent([sys.executable, "-c", "import sys; print('step 1', flush=True); sys.exit(3)"],
                  hang_timeout_seconds=5, max_restarts=2, poll_interval_seconds=0.05)
    final = agent.run()
    assert final.state == WorkerState.FAILED and final.restarts == 2 and final.last_exit_code == 3


def _fake_worker(steps, crash_at=None, marker=None, delay=0.05):
    body = (
        "import os, sys, time\n"
        f"marker = {marker!r}\n"
        f"for s in range(1, {steps} + 1):\n"
        "    print(f'step {s}', flush=True)\n"
        f"    time.sleep({delay})\n"
        f"    if {crash_at!r} is not None and s == {crash_at!r} and not os.path.exists(marker):\n"
        "        open(marker, 'w').close(); sys.exit(7)\n"
    )
    return [sys.executable, "-c", body]


def test_manager_turns_one_failure_into_a_job_wide_restart(tmp_path):
    mgr = Manager(heartbeat_timeout_seconds=5).start()
    host, port = mgr.address
    results = {}

    def run(wid, cmd):
        client = ManagerClient(host, port, worker_id=wid)
        agent = Agent(cmd, hang_timeout_seconds=10, max_restarts=3, poll_interval_seconds=0.02,
                      report_fn=client.report)
        results[wid] = (agent.run(), agent)

    threads = [
        threading.Thread(target=run, args=("w0", _fake_worker(60, crash_at=10, marker=str(tmp_path / "m")))),
        threading.Thread(target=run, args=("w1", _fake_worker(60))),
    ]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    try:
        assert results["w0"][0].state == WorkerState.FINISHED and results["w1"][0].state == WorkerState.FINISHED
        # w0 crashed once; w1 was healthy but restarted with it.
        assert results["w0"][1].restarts == 1 and results["w1"][1].restarts == 1
        assert any("restart requested by the manager" in h.reason for h in results["w1"][1].history)
        assert mgr.generation == 1 and "w0 crashed" in mgr.events[0][2]
    finally:
        mgr.stop()


def test_manager_hierarchy_heartbeats_and_stragglers():
    top = Manager(manager_id="global").start()
    replica = Manager(upstream=top.address, manager_id="replica0", heartbeat_timeout_seconds=0.3,
                      straggler_ratio=0.5).start()
    try:
        host, port = replica.address
        dropped = []
        fast = ManagerClient(host, port, worker_id="fast")
        slow = ManagerClient(host, port, worker_id="slow")
        lossy = ManagerClient(host, port, worker_id="lossy", drop_fn=lambda m: dropped.append(m) or len(dropped) > 1)
        rep = lambda state, step: types.SimpleNamespace(state=WorkerState(state), step=step, restarts=0, reason="")
        for c in (fast, slow, lossy):
            c.report(rep("starting", -1))
        for i in range(1, 6):
            fast.report(rep("running", 10 * i))
            slow.report(rep("running", 2 * i))
            lossy.report(rep("running", 10 * i))     # every message after the first is lost
            time.sleep(0.1)
        status = fast.send({"type": "status"})
        assert status["stragglers"] == ["slow"]
        assert status["missing_heartbeats"] == ["lossy"]
        # A failure reported to the replica manager reaches the global manager ...
        fast.report(rep("hung", 50))
        assert replica.generation == 1 and top.generation == 1
        # ... and a generation raised at the top (another replica failed) flows down on poll.
        ManagerClient(*top.address, worker_id="replica1").send(
            {"type": "report", "worker_id": "replica1", "state": "crashed", "step": 3})
        replica.poll_upstream()
        assert replica.generation == 2
        assert slow.report(rep("running", 12)) == "restart"
    finally:
        replica.stop()
        top.stop()


def test_device_monitor_with_fake_nvml():
    class FakeNvml:
        def __init__(self):
            self.util = [80.0, 90.0]
            self.inits = 0

        def nvmlInit(self):  # pylint: disable=invalid-name
            self.inits += 1

        def nvmlDeviceGetCount(self):  # pylint: disable=invalid-name
            return len(self.util)

        def nvmlDeviceGetHandleByIndex(self, i):  # pylint: disable=invalid-name
            return i

        def nvmlDeviceGetUtilizationRates(self, h):  # pylint: disable=invalid-name
            return types.SimpleNamespace(gpu=self.util[h], memory=10.0)

        def nvmlDeviceGetMemoryInfo(self, h):  # pylint: disable=invalid-name
            return types.SimpleNamespace(used=40e9, total=180e9)

    fake = FakeNvml()
    cfg = DeviceMonitor.default_config().set(
        monitor_client=GPUMonitorClient.default_config().set(nvml=lambda: fake), check_interval_in_sec=0.05)
    mon = cfg.instantiate()
    mon.start_monitoring()
    try:
        assert not mon.is_host_idle() and len(mon.last_metrics()) == 2
        fake.util = [0.0, 1.0]
        time.sleep(0.3)
        assert mon.is_host_idle()
        assert abs(mon.last_metrics()[0]["mem_used_frac"] - 40 / 180) < 1e-6
    finally:
        mon.stop_monitoring()
    assert fake.inits == 1


def test_liveness_monitor_and_status_server(tmp_path):
    mon = LivenessMonitor.default_config().set(
        summary_dir=str(tmp_path), max_timeout_seconds=0.3, max_start_seconds=0.3).instantiate()
    with pytest.raises(RuntimeError):
        mon.ping()
    mon.reset()
    assert mon.ping()
    (tmp_path / "events.jsonl").write_text("x")
    assert mon.ping()
    time.sleep(0.5)
    assert not mon.ping()          # no new summaries for longer than the timeout
    (tmp_path / "events.jsonl").write_text("xy")
    assert mon.ping()

    server = StatusHTTPServer(0)
    server.start()
    try:
        body = urllib.request.urlopen(f"http://127.0.0.1:{server.port}/", timeout=5).read().decode()
        assert "status-server" in body or "Thread" in body
    finally:
        server.stop()
