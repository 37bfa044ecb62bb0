"""Worker -> replica manager -> global manager hierarchy, hang detection and straggler detection.

Everything runs as threads and sockets on the CPU; failures are reports that the test sends."""

from axlearn_b200.ft.manager_server import GlobalManager, ReplicaManager, WorkerClient
from axlearn_b200.ft.monitor import STRAGGLER_CONFIRMED, STRAGGLER_POTENTIAL, StatusMonitor, StragglerMonitor


def _job(num_replicas=2, workers_per_replica=2):
    gm = GlobalManager(num_replicas=num_replicas).start()
    rms = [ReplicaManager(r, global_address=gm.address).start() for r in range(num_replicas)]
    clients = [[WorkerClient(rm.address, replica_id=r, worker_id=w, hostname=f"host-{r}-{w}")
                for w in range(workers_per_replica)] for r, rm in enumerate(rms)]
    return gm, rms, clients


def _stop(gm, rms):
    for rm in rms:
        rm.stop()
    gm.stop()


def test_one_crash_restarts_every_worker_exactly_once():
    gm, rms, clients = _job()
    try:
        for row in clients:
            for c in row:
                assert c.report_status(step=10) is None
        for rm in rms:
            rm.report_replica_status()
        assert gm.get_global_status() == {"replicas": 2, "expected_replicas": 2, "workers": 4, "global_restart_count": 0}
        # Worker (1, 0) crashes; worker (1, 1), whose collective died with it, reports a crash too.
        clients[1][0].report_status(step=10, state="crashed", reason="exit code 1")
        clients[1][1].report_status(step=10, state="crashed", reason="NCCL error")
        assert gm.global_restart_count == 1  # the second request carried a stale count
        assert [rm.restart_count for rm in rms] == [1, 1]
        # Healthy workers learn about it with their next report and restart; then they are quiet.
        assert clients[0][0].report_status(step=11) == "restart"
        assert clients[0][0].restart_count == 1
        assert clients[0][0].report_status(step=0) is None
        assert clients[0][1].report_status(step=11) == "restart"
        # A later, separate failure starts generation 2.
        for c in clients[1]:
            c.restart_count = 1
        clients[1][1].report_status(step=3, state="hung", reason="no progress")
        assert gm.global_restart_count == 2
    finally:
        _stop(gm, rms)


def test_pod_shutdown_and_explicit_request_go_to_the_global_manager():
    gm, rms, clients = _job()
    try:
        for rm in rms:
            rm.report_replica_status()
        reply = clients[0][1].report_pod_shutdown("preempted")
        assert reply["acknowledged"] and gm.global_restart_count == 1 and len(gm.shutdowns) == 1
        stale = clients[1][0].request_global_restart("late news")  # still at count 0
        assert not stale["acknowledged"] and gm.global_restart_count == 1
        clients[1][0].restart_count = 1
        assert clients[1][0].request_global_restart("new failure")["acknowledged"]
        assert gm.global_restart_count == 2 and all(rm.restart_count == 2 for rm in rms)
    finally:
        _stop(gm, rms)


def test_hang_detection_restarts_all_replicas():
    gm, rms, clients = _job()
    clock = {"t": 1000.0}
    try:
        for row in clients:
            for c in row:
                c.report_status(step=5)
        monitors = [StatusMonitor(replica_manager=rm) for rm in rms]
        top = StatusMonitor(global_manager=gm, hang_threshold_seconds=60, now_fn=lambda: clock["t"])
        for m in monitors:
            m.run_once()
        import time as _time

        clock["t"] = _time.time() + 10
        top.run_once()
        assert not top.restarts_triggered
        # Replica 0 keeps reporting the same step (alive but stuck); replica 1 advances.
        for c in clients[0]:
            c.report_status(step=5)
        for c in clients[1]:
            c.report_status(step=6)
        for m in monitors:
            m.run_once()
        clock["t"] = _time.time() + 120
        # Replica 1 advanced "just now" relative to its own reports, but 120 s later both look
        # stale; refresh replica 1 so that only replica 0 hangs.
        for c in clients[1]:
            c.report_status(step=7)
        rms[1].workers[0]["last_update"] = clock["t"]
        rms[1].workers[1]["last_update"] = clock["t"]
        for m in monitors:
            m.run_once()
        assert top.count_hanging_replicas(gm.get_detailed_global_status()["replicas"]) == 1
        top.run_once()
        assert len(top.restarts_triggered) == 1 and gm.global_restart_count == 1
        assert all(rm.restart_count == 1 for rm in rms)
    finally:
        _stop(gm, rms)


def _status(utils):
    return {"replicas": {0: {"workers": [
        {"worker_identity": {"worker_id": i, "hostname": f"h{i}"}, "tensorcore_util": u} for i, u in enumerate(utils)]}}}


def test_straggler_monitor_uses_median_absolute_deviation_and_sustained_duration():
    clock = {"t": 0.0}
    lines = []
    mon = StragglerMonitor(sensitivity=5.0, sustained_duration_seconds=100, now_fn=lambda: clock["t"], log_fn=lines.append)
    healthy = [91.0, 90.0, 89.5, 90.5, 90.2, 89.8, 90.1]
    assert mon.run_check(_status(healthy + [90.3])) == []
    slow = healthy + [40.0]
    assert mon.run_check(_status(slow)) == []          # an outlier, but only just now
    clock["t"] = 55.0
    rep = mon.run_check(_status(slow))
    assert [r["label"] for r in rep] == [STRAGGLER_POTENTIAL] and rep[0]["worker_id"] == 7
    clock["t"] = 120.0
    rep = mon.run_check(_status(slow))
    assert [r["label"] for r in rep] == [STRAGGLER_CONFIRMED] and rep[0]["modified_z"] < -5
    assert "CONFIRMED STRAGGLER" in lines[-1]
    # Recovery clears the history: the clock starts again.
    assert mon.run_check(_status(healthy + [90.0])) == []
    clock["t"] = 130.0
    assert mon.run_check(_status(slow)) == []
    # Too few workers, identical workers, unavailable readings.
    assert StragglerMonitor().run_check(_status([90, 10, 90])) == []
    assert StragglerMonitor().run_check(_status([90, 90, 90, 90, 90])) == []
    assert StragglerMonitor().run_check(_status([-1, -1, -1, -1, 50])) == []
