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
