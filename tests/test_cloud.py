"""Quota, scheduler, bundler, bastion and the command line (all on local directories)."""

import datetime
import json
import os
import sys
import tarfile
import time

import pytest

from axlearn_b200.cli.main import main as cli_main
from axlearn_b200.cloud.common import quota
from axlearn_b200.cloud.common.bastion import Bastion, BastionDirectory, JobState
from axlearn_b200.cloud.common.bundler import TarBundler, get_bundler_config
from axlearn_b200.cloud.common.cleaner import UnschedulableCleaner
from axlearn_b200.cloud.common.job import Job
from axlearn_b200.cloud.common.job_types import JobMetadata, JobSpec
from axlearn_b200.cloud.common.scheduler import JobScheduler, ProjectJobSorter, TierScheduler
from axlearn_b200.common.config import config_for_function

T0 = datetime.datetime(2026, 1, 1)


def _meta(user, project, minutes, gpus, priority=5):
    return JobMetadata(user_id=user, project_id=project, creation_time=T0 + datetime.timedelta(minutes=minutes),
                       resources={"b200": gpus}, priority=priority)


def _quota_file(tmp_path, tiers=({"b200": 16},), shares=None):
    path = tmp_path / "quota.json"
    path.write_text(json.dumps({
        "total_resources": list(tiers),
        "project_resources": shares or {"a": {"b200": 0.5}, "b": {"b200": 0.5}},
        "project_membership": {"a": ["alice", "al.*"], "b": ["bob"]}}))
    return str(path)


def test_quota_file_and_membership(tmp_path):
    info = quota.get_resource_limits(_quota_file(tmp_path))
    assert info.total_resources == [{"b200": 16}]
    assert info.user_projects("alfred") == ["a"] and info.user_projects("bob") == ["b"]
    assert quota.get_user_projects(_quota_file(tmp_path), "carol") == []


def test_sorter_priority_then_fair_share_then_age():
    jobs = {"a1": _meta("alice", "p", 0, 8), "a2": _meta("alice", "p", 1, 8), "b1": _meta("bob", "p", 2, 8),
            "urgent": _meta("bob", "p", 9, 8, priority=1)}
    order = [j for j, _ in ProjectJobSorter.default_config().instantiate().sort(jobs)]
    # bob already holds the urgent job, so alice's first job precedes bob's next; then they alternate.
    assert order == ["urgent", "a1", "a2", "b1"] or order == ["urgent", "a1", "b1", "a2"]
    fifo = [j for j, _ in ProjectJobSorter.default_config().set(use_user_usage=False).instantiate().sort(jobs)]
    assert fifo == ["urgent", "a1", "a2", "b1"]


def test_tier_scheduler_fairness_tiers_and_over_limits():
    sched = TierScheduler.default_config().instantiate()
    jobs_a = [("a1", _meta("alice", "a", 0, 8)), ("a2", _meta("alice", "a", 1, 8)), ("a3", _meta("alice", "a", 2, 8))]
    jobs_b = [("b1", _meta("bob", "b", 3, 8))]
    res = sched.schedule(resource_limits=[{"b200": 16}, {"b200": 8}],
                         project_quotas={"a": {"b200": 1}, "b": {"b200": 1}},
                         project_jobs={"a": jobs_a, "b": jobs_b})
    v = res.job_verdicts
    # Both projects get their share of the reserved tier first; a's second job spills to tier 1;
    # its third finds nothing left.
    assert v["a1"].metadata["tier"] == 0 and v["b1"].metadata["tier"] == 0
    assert v["a2"].metadata["tier"] == 1
    assert not v["a3"] and v["a3"].over_limits == {"b200"}
    assert res.project_usages == {"a": {"b200": 16}, "b": {"b200": 8}}
    assert res.project_limits["a"]["b200"] == pytest.approx(12.0)
    # A job larger than the whole cluster does not block the smaller one behind it.
    res = sched.schedule(resource_limits=[{"b200": 8}], project_quotas={"a": {"b200": 1}},
                         project_jobs={"a": [("huge", _meta("alice", "a", 0, 64)), ("small", _meta("alice", "a", 1, 8))]})
    assert not res.job_verdicts["huge"] and res.job_verdicts["small"]


def test_job_scheduler_reads_quota_and_dry_run(tmp_path):
    cfg = JobScheduler.default_config().set(
        quota=config_for_function(quota.get_resource_limits).set(path=_quota_file(tmp_path, tiers=({"b200": 8},))))
    jobs = {"a1": _meta("alice", "a", 0, 8), "b1": _meta("bob", "b", 1, 8)}
    res = cfg.instantiate().schedule(jobs)
    assert res.job_verdicts["a1"] and not res.job_verdicts["b1"]
    assert all(cfg.instantiate().schedule(jobs, dry_run=True).job_verdicts.values())


def test_job_retries(tmp_path):
    marker = tmp_path / "tries"

    class Flaky(Job):
        def _execute(self):
            n = int(marker.read_text()) if marker.exists() else 0
            marker.write_text(str(n + 1))
            if n < 2:
                raise RuntimeError("not yet")
            return "ok"

    assert Flaky.default_config().set(name="flaky", max_tries=3, retry_interval=0.0).instantiate().execute() == "ok"
    marker.unlink()
    with pytest.raises(RuntimeError):
        Flaky.default_config().set(name="flaky", max_tries=2, retry_interval=0.0).instantiate().execute()


def test_tar_bundler(tmp_path):
    src = tmp_path / "src"
    (src / "pkg" / "__pycache__").mkdir(parents=True)
    (src / "pkg" / "mod.py").write_text("x = 1\n")
    (src / "pkg" / "__pycache__" / "mod.pyc").write_text("junk")
    (src / ".git").mkdir()
    (src / ".git" / "HEAD").write_text("ref")
    cfg = get_bundler_config(bundler_type="tar", spec=[f"remote_dir={tmp_path / 'bundles'}"])
    out = cfg.instantiate().bundle("job1", src_dir=str(src))
    with tarfile.open(out) as tar:
        assert tar.getnames() == ["pkg/mod.py"]
    assert "tar -xzf" in TarBundler.install_command(out, dest="/tmp/x")
    with pytest.raises(NotImplementedError):
        get_bundler_config(bundler_type="no-such-bundler")


def _bastion(tmp_path, gpus=8, cleaner=False, shares=None):
    sched = JobScheduler.default_config().set(
        quota=config_for_function(quota.get_resource_limits).set(
            path=_quota_file(tmp_path, tiers=({"b200": gpus},), shares=shares)))
    cfg = Bastion.default_config().set(root_dir=str(tmp_path / "bastion"), scheduler=sched, update_interval_seconds=0.05,
                                       termination_grace_seconds=2.0, publish_events=True)
    if cleaner:
        cfg.cleaner = UnschedulableCleaner.default_config().set(scheduler=sched)
    return cfg.instantiate()


def _spec(name, command, meta, cleanup=None):
    return JobSpec(version=1, name=name, command=command, cleanup_command=cleanup, env_vars={"FOO": "bar"}, metadata=meta)


def _wait(bastion, predicate, timeout=20.0):
    deadline = time.time() + timeout
    while time.time() < deadline:
        bastion.execute_once()
        if predicate():
            return
        time.sleep(0.05)
    raise AssertionError("timed out")


def test_bastion_runs_jobs_to_completion_with_cleanup(tmp_path):
    b = _bastion(tmp_path)
    out = tmp_path / "out.txt"
    py = sys.executable
    b.directory.submit_job("j1", job_spec=_spec(
        "j1", f"{py} -c \"import os; open(r'{out}', 'w').write(os.environ['FOO'] + os.environ['BASTION_JOB_NAME'])\"",
        _meta("alice", "a", 0, 8), cleanup=f"{py} -c \"open(r'{out}.clean', 'w').write('done')\""))
    done = lambda: os.path.exists(tmp_path / "bastion" / "jobs" / "complete" / "j1")
    _wait(b, done)
    assert out.read_text() == "barj1" and (tmp_path / "out.txt.clean").read_text() == "done"
    st = b.directory.get_job_state("j1")
    assert st.state == JobState.COMPLETED and st.metadata["returncode"] == 0
    assert not os.path.exists(tmp_path / "bastion" / "jobs" / "active" / "j1")
    import json
    events = [json.loads(l) for l in (tmp_path / "bastion" / "events.jsonl").read_text().splitlines()]
    states = [e["state"] for e in events if e["job_name"] == "j1"]
    assert states[0] in ("PENDING", "ACTIVE", "pending", "active") and states[-1].lower() == "completed"
    assert len(states) == len(set(states))                      # one event per state change
    b.shutdown()


def test_bastion_queues_preempts_and_cancels(tmp_path):
    # Project b has no quota of its own: it runs on spare capacity only.
    b = _bastion(tmp_path, gpus=8, shares={"a": {"b200": 1.0}, "b": {"b200": 0.0}})
    py = sys.executable
    sleeper = f"{py} -c \"import time; time.sleep(60)\""
    b.directory.submit_job("low", job_spec=_spec("low", sleeper, _meta("bob", "b", 0, 8, priority=5)))
    b.execute_once()
    assert b.directory.get_job_state("low").state == JobState.ACTIVE
    # A second job of the same size waits ...
    b.directory.submit_job("waits", job_spec=_spec("waits", sleeper, _meta("bob", "b", 1, 8)))
    b.execute_once()
    assert b.directory.get_job_state("waits").state == JobState.PENDING
    # ... and a job of the project that owns the quota pre-empts the running one.
    b.directory.submit_job("fair", job_spec=_spec("fair", sleeper, _meta("alice", "a", 2, 8)))
    b.execute_once()
    b.execute_once()
    states = {n: b.directory.get_job_state(n).state for n in ("low", "waits", "fair")}
    assert states["fair"] == JobState.ACTIVE and states["low"] == JobState.PENDING, states
    assert b.directory.get_job_state("low").metadata.get("preempted")
    # Cancelling ends the job and lets the next one in.
    b.directory.cancel_job("fair")
    _wait(b, lambda: os.path.exists(tmp_path / "bastion" / "jobs" / "complete" / "fair"))
    _wait(b, lambda: b.directory.get_job_state("low").state == JobState.ACTIVE)
    b.shutdown()


def test_unschedulable_jobs_are_swept(tmp_path):
    b = _bastion(tmp_path, gpus=8, cleaner=True)
    b.directory.submit_job("huge", job_spec=_spec("huge", "true", _meta("alice", "a", 0, 64)))
    b.execute_once()
    st = b.directory.get_job_state("huge")
    assert st.state == JobState.COMPLETED and st.metadata["unschedulable"]
    b.shutdown()


def test_cli_bastion_round_trip(tmp_path, capsys):
    root = str(tmp_path / "bastion")
    q = _quota_file(tmp_path)
    marker = tmp_path / "cli.txt"
    assert cli_main(["bastion", "submit", "--root_dir", root, "--name", "c1", "--project", "a", "--user", "alice",
                     "--resources", "b200=8", "--command",
                     f"{sys.executable} -c \"open(r'{marker}', 'w').write('ran')\""]) == 0
    assert cli_main(["bastion", "list", "--root_dir", root]) == 0
    assert '"c1"' in capsys.readouterr().out
    assert cli_main(["bastion", "start", "--root_dir", root, "--quota_file", q, "--interval", "0.2",
                     "--max_iterations", "8"]) == 0
    assert marker.read_text() == "ran"
    assert cli_main(["bastion", "state", "--root_dir", root, "--name", "c1"]) == 0
    assert "COMPLETED" in capsys.readouterr().out
    assert cli_main(["bundle", "--name", "b1", "--remote_dir", str(tmp_path / "bundles"), "--src_dir",
                     os.path.dirname(os.path.abspath(__file__))]) == 0
    assert os.path.exists(tmp_path / "bundles" / "b1.tar.gz")
    with pytest.raises(SystemExit):
        cli_main(["bastion", "submit", "--root_dir", root])
