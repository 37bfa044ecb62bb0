"""GKE runner job against in-memory Kubernetes / container APIs (reference behaviour:
axlearn/cloud/gcp/runners/gke.py:549-889, runners/utils.py)."""

import pytest

from axlearn_b200.cloud.common.event_queue import InMemoryQueueClient
from axlearn_b200.cloud.gcp.job import GKEJob
from axlearn_b200.cloud.gcp.jobset_utils import A4HighReplicatedJob
from axlearn_b200.cloud.gcp.node_pool_provisioner import GPUNodePoolProvisioner
from axlearn_b200.cloud.gcp.runners import gke
from axlearn_b200.cloud.gcp.runners.utils import should_recreate_job
from tests.test_cloud_gcp_orchestration import FakeContainer, FakeKubernetes

Status = gke.GKERunnerJob.Status


@pytest.mark.parametrize("tier,reservation,processor,pending,want", [
    ("0", "res", "gpu", False, False), ("1", "res", "gpu", False, True), ("disabled", "res", "gpu", False, False),
    ("0", None, "gpu", False, False), ("0", None, "gpu", True, True), ("1", None, "gpu", True, False),
    ("1", "res", None, False, False), ("1", "res", "cpu", True, False), (0, None, "tpu", True, True),
])
def test_should_recreate_job(tier, reservation, processor, pending, want):
    assert should_recreate_job(tier, reservation, processor, is_pending=pending) is want


class ScriptedKubernetes(FakeKubernetes):
    """After creation the JobSet's status follows ``script`` (one entry per read; the last repeats)."""

    def __init__(self, script):
        super().__init__()
        self.script, self.created, self.deleted = list(script), 0, 0

    def create_jobset(self, namespace, body):
        self.created += 1
        return super().create_jobset(namespace, body)

    def delete_jobset(self, namespace, name):
        self.deleted += 1
        super().delete_jobset(namespace, name)

    def get_jobset(self, namespace, name):
        js = super().get_jobset(namespace, name)
        if js is None:
            return None
        step = self.script.pop(0) if len(self.script) > 1 else self.script[0]
        return dict(js, status=step)


def _status(ready=0, succeeded=0, failed=0, conditions=()):
    return {"replicatedJobsStatus": [{"name": "job", "ready": ready, "succeeded": succeeded, "failed": failed}],
            "conditions": [{"type": t, "status": "True", "reason": "r"} for t in conditions]}


def _runner(api, *, environ=None, container=None, provision=False, reservation=None, spot=False, bundler=None, **kw):
    builder = A4HighReplicatedJob.default_config().set(command="python -m x", image="img:1", num_nodes=2,
                                                       reservation=reservation, enable_spot=spot)
    cfg = gke.GKERunnerJob.default_config().set(
        name="exp", inner=GKEJob.default_config().set(builder=builder), project="proj", zone="us-central1-b", cluster="c1",
        status_interval_seconds=7, **kw)
    if provision:
        cfg.pre_provisioner = GPUNodePoolProvisioner.default_config().set(
            project="proj", zone="us-central1-b", cluster="c1", retry_interval=0, wait_timeout=5)
    queue, naps = InMemoryQueueClient(), []
    job = cfg.instantiate(api=api, container_api=container, event_publisher=queue, sleep=naps.append,
                          environ=environ if environ is not None else {}, bundler=bundler)
    return job, queue, naps


def test_start_monitor_and_finish():
    api = ScriptedKubernetes([_status(), _status(ready=1), _status(ready=1), _status(succeeded=1, conditions=["Completed"])])
    job, queue, naps = _runner(api)
    assert job.execute() == Status.COMPLETED
    assert api.created == 1 and api.deleted == 0
    assert [(e.state, e.details) for e in queue.events] == [
        ("STARTING", "Cloud build finished"), ("STARTING", "Provisioning resources"), ("STARTING", "Job is starting"),
        ("RUNNING", "Job is running"), ("SUCCEEDED", "Job succeeds")]
    assert naps == [7] * 4 and "time_to_running" in job.timings and not job.is_running


def test_failed_condition_and_child_failures():
    api = ScriptedKubernetes([_status(failed=1), _status(failed=1, conditions=["Failed"])])
    job, queue, _ = _runner(api)
    assert job.execute() == Status.FAILED
    assert queue.events[-1].state == "FAILED" and queue.events[-2].details == "Job is starting"


def test_version_bump_relaunches():
    api = ScriptedKubernetes([_status(ready=1)])
    env = {}
    job, _, _ = _runner(api, environ=env, max_polls=2)
    assert job.execute() == Status.READY and job.is_running
    env[gke.BASTION_JOB_VERSION_ENV_VAR] = "3"
    # The deployed JobSet carries no version: it is deleted, then started again by the next poll.
    assert job._get_status() == Status.UPDATING   # pylint: disable=protected-access
    job.execute()
    assert api.deleted == 1 and api.created == 2


def test_build_failure_aborts():
    class BadBundler:
        def wait_until_finished(self, name):
            raise RuntimeError(f"build {name} failed")

    api = ScriptedKubernetes([_status()])
    job, queue, _ = _runner(api, bundler=BadBundler())
    assert job.execute() is None and api.created == 0 and queue.events == []


def test_tier_change_reschedules_and_replaces_pools():
    # The job was provisioned on a reservation (tier 0); the bastion then moves it to tier 1.
    container = FakeContainer(ready_after=0)
    env = {"BASTION_TIER": "0"}
    api = ScriptedKubernetes([_status(ready=1)])
    job, _, _ = _runner(api, environ=env, container=container, provision=True, reservation="res", max_polls=2)
    assert job.execute() == Status.READY
    (pool,) = container.created
    assert container.deleted == []
    env["BASTION_TIER"] = "1"
    assert job._get_status() == Status.RESCHEDULED   # pylint: disable=protected-access
    job.execute()
    # Poll 1 deleted the JobSet and the reservation-backed pool; poll 2 found nothing and started over.
    assert api.deleted == 1 and container.deleted == [pool] and api.created == 2 and container.created == [pool, pool]
    # A tier-0 job that runs on spot nodes keeps running (recreated only while pending).
    env["BASTION_TIER"] = "0"
    api2 = ScriptedKubernetes([_status(ready=1), _status()])
    job2, _, _ = _runner(api2, environ=env, spot=True, max_polls=2)
    assert job2.execute() == Status.READY
    assert job2._get_status() == Status.RESCHEDULED   # pending now  # pylint: disable=protected-access


def test_spec_inference_helpers():
    spec = {"replicatedJobs": [{"replicas": 2, "template": {"spec": {"template": {
        "metadata": {"labels": {gke.BASTION_JOB_VERSION_LABEL: "4"}},
        "spec": {"nodeSelector": {"cloud.google.com/reservation-name": "r"},
                 "containers": [{"resources": {"limits": {"nvidia.com/gpu": 8}}}]}}}}}]}
    assert gke.infer_reservation(spec) == "r" and gke.infer_processor_type(spec) == "gpu"
    assert gke.infer_job_version(spec) == 4 and gke.infer_job_count(spec) == 2
    assert gke.infer_reservation({"replicatedJobs": [{}]}) is None
    pools = [{"name": "a", "config": {"reservationAffinity": {"key": "compute.googleapis.com/reservation-name", "values": ["r"]}}},
             {"name": "b", "config": {"taints": [{"key": "cloud.google.com/gke-spot", "value": "true", "effect": "NO_SCHEDULE"}]}}]
    assert [p["name"] for p in gke.mismatched_node_pools(pools, tier="0")] == ["b"]
    assert [p["name"] for p in gke.mismatched_node_pools(pools, tier=2)] == ["a"]
