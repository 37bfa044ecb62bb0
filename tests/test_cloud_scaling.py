"""Scaling specs, replica manager, command patcher."""

import datetime

from axlearn_b200.cloud.common import scaling
from axlearn_b200.cloud.common.job_types import JobMetadata, JobSpec, ScalingSpec, Topology, deserialize_jobspec, serialize_jobspec
from axlearn_b200.cloud.common.replica_manager import FileReplicaManager
from axlearn_b200.cloud.common.user_command_patcher import EnvPrefixPatcher


def test_aggregates():
    specs = [ScalingSpec(min_replicas=2, max_replicas=4, resources_per_replica={"b200": 8}, topology_per_replica="8x1", name="train"),
             ScalingSpec(min_replicas=1, max_replicas=1, resources_per_replica={"b200": 8, "cpu": 4})]
    assert scaling.aggregate_min_resources(specs) == {"b200": 24, "cpu": 4}
    assert scaling.aggregate_topology(specs) == [Topology(topology="8x1", replicas=2)]
    assert scaling.aggregate_min_resources([]) == {} and scaling.aggregate_topology(specs[1:]) == []


def test_jobspec_round_trip_with_scaling_specs(tmp_path):
    meta = JobMetadata(user_id="u", project_id="p", creation_time=datetime.datetime(2024, 1, 2), resources={"b200": 16},
                       scaling_specs=[ScalingSpec(min_replicas=1, max_replicas=3, resources_per_replica={"b200": 8}, name="g")])
    spec = JobSpec(version=1, name="j", command="true", cleanup_command=None, env_vars=None, metadata=meta)
    path = str(tmp_path / "j")
    serialize_jobspec(spec, path)
    assert deserialize_jobspec(path) == spec
    plain = JobSpec(version=1, name="j", command="true", cleanup_command=None, env_vars=None,
                    metadata=JobMetadata(user_id="u", project_id="p", creation_time=datetime.datetime(2024, 1, 2), resources={}))
    serialize_jobspec(plain, path)
    assert deserialize_jobspec(path).metadata.scaling_specs is None


def test_file_replica_manager(tmp_path):
    m = FileReplicaManager.default_config().set(root_dir=str(tmp_path / "replicas")).instantiate()
    assert m.get_desired_replicas("job") is None
    m.set_desired_replicas("job", {"train": 3})
    m.set_granted_replicas("job", {"train": 2})
    other = FileReplicaManager.default_config().set(root_dir=str(tmp_path / "replicas")).instantiate()
    other.refresh()
    assert other.get_desired_replicas("job") == {"train": 3} and other.get_granted_replicas("job") == {"train": 2}
    (tmp_path / "replicas" / "broken.json").write_text("{")
    other.refresh()                                       # a half-written file is skipped
    assert other.get_desired_replicas("broken") is None


def test_env_prefix_patcher():
    p = EnvPrefixPatcher.default_config().set(env_vars={"A": "1"}).instantiate()
    assert p.patch("python x.py", env_vars={"B": "two words"}) == "A=1 B='two words' python x.py"
    assert EnvPrefixPatcher.default_config().instantiate().patch("cmd") == "cmd"


def test_elastic_jobs_get_replicas_as_quota_allows():
    from axlearn_b200.cloud.common.quota import QuotaInfo
    from axlearn_b200.cloud.common.scheduler import JobScheduler

    def meta(project, t, resources, specs=None, priority=5):
        return JobMetadata(user_id="u", project_id=project, creation_time=datetime.datetime(2024, 1, 1, 0, t),
                           resources=resources, priority=priority, scaling_specs=specs)

    quota = QuotaInfo(total_resources=[{"b200": 40}], project_resources={"a": {"b200": 0.5}, "b": {"b200": 0.5}},
                      project_membership={})
    sched = JobScheduler.default_config().set(quota=lambda: quota).instantiate()
    elastic = [ScalingSpec(min_replicas=1, max_replicas=4, resources_per_replica={"b200": 8}, name="train")]
    jobs = {"el": meta("a", 0, {"b200": 8}, elastic), "fixed": meta("b", 1, {"b200": 16})}
    # Nothing asked beyond the minimum: one replica granted, no slots in the verdicts.
    r = sched.schedule(jobs)
    assert set(r.job_verdicts) == {"el", "fixed"} and r.job_verdicts["el"].metadata["granted_replicas"] == {"train": 1}
    assert "granted_replicas" not in r.job_verdicts["fixed"].metadata
    # Four replicas wanted: 8 (base) + 16 (fixed) leave 16 of 40, i.e. two more replicas.
    r = sched.schedule(jobs, desired_replicas={"el": {"train": 4}})
    assert set(r.job_verdicts) == {"el", "fixed"}
    assert r.job_verdicts["el"].metadata["granted_replicas"] == {"train": 3} and r.job_verdicts["fixed"]
    assert r.project_usages["a"]["b200"] == 24
    # A request beyond max_replicas is capped.
    big = QuotaInfo(total_resources=[{"b200": 400}], project_resources={"a": {"b200": 1.0}}, project_membership={})
    r = JobScheduler.default_config().set(quota=lambda: big).instantiate().schedule(
        {"el": jobs["el"]}, desired_replicas={"el": {"train": 9}})
    assert r.job_verdicts["el"].metadata["granted_replicas"] == {"train": 4}
    # A parent that does not fit drops its slots.
    tiny = QuotaInfo(total_resources=[{"b200": 4}], project_resources={"a": {"b200": 1.0}}, project_membership={})
    r = JobScheduler.default_config().set(quota=lambda: tiny).instantiate().schedule(
        {"el": jobs["el"]}, desired_replicas={"el": {"train": 2}})
    assert set(r.job_verdicts) == {"el"} and not r.job_verdicts["el"]


def test_bastion_reports_granted_replicas(tmp_path):
    import json

    from axlearn_b200.cloud.common.bastion import Bastion, BastionDirectory
    from axlearn_b200.cloud.common.scheduler import JobScheduler
    from axlearn_b200.common.config import config_for_function
    from axlearn_b200.cloud.common import quota as quota_lib

    quota_file = tmp_path / "quota.json"
    quota_file.write_text(json.dumps({"total_resources": {"b200": 24}, "project_resources": {"p": {"b200": 1.0}}}))
    root = str(tmp_path / "bastion")
    replicas_dir = str(tmp_path / "replicas")
    manager_cfg = FileReplicaManager.default_config().set(root_dir=replicas_dir)
    manager_cfg.instantiate().set_desired_replicas("el", {"default": 4})
    sched = JobScheduler.default_config().set(quota=config_for_function(quota_lib.get_resource_limits).set(path=str(quota_file)))
    bastion = Bastion.default_config().set(root_dir=root, scheduler=sched, update_interval_seconds=0.01,
                                           replica_manager=manager_cfg).instantiate()
    meta = JobMetadata(user_id="u", project_id="p", creation_time=datetime.datetime(2024, 1, 1), resources={"b200": 8},
                       scaling_specs=[ScalingSpec(min_replicas=1, max_replicas=8, resources_per_replica={"b200": 8})])
    BastionDirectory.default_config().set(root_dir=root).instantiate().submit_job(
        "el", job_spec=JobSpec(version=1, name="el", command="sleep 0.2", cleanup_command=None, env_vars=None, metadata=meta))
    bastion.execute(max_iterations=2)
    # 24 GPUs: the base replica and two more of the four wanted.
    assert manager_cfg.instantiate().get_granted_replicas("el") == {"default": 3}
