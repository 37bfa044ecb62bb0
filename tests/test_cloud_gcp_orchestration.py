"""GKE orchestration against fakes: replicated-job builders, JobSet assembly and status, node-pool
provisioning, goodput recorder."""

import time

import pytest

from axlearn_b200.cloud.gcp import node_pool
from axlearn_b200.cloud.gcp.job import GKEJob, JobSetStatus, jobset_status
from axlearn_b200.cloud.gcp.jobset_utils import (
    A3UltraReplicatedJob,
    A4HighReplicatedJob,
    CompositeReplicatedJob,
    EphemeralDiskMount,
    GCSFuseMount,
    GPUReplicatedJob,
    HostMount,
    JobDependency,
)
from axlearn_b200.cloud.gcp.node_pool_provisioner import GPUNodePoolProvisioner
from axlearn_b200.common import measurement


class FakeKubernetes:
    def __init__(self):
        self.jobsets = {}

    def create_jobset(self, namespace, body):
        self.jobsets[(namespace, body["metadata"]["name"])] = body
        return body

    def get_jobset(self, namespace, name):
        return self.jobsets.get((namespace, name))

    def delete_jobset(self, namespace, name):
        self.jobsets.pop((namespace, name), None)


class FakeContainer:
    """Pools become RUNNING ``ready_after`` status reads after their creation."""

    def __init__(self, ready_after=2, fail=()):
        self.pools, self.reads, self.ready_after, self.fail = {}, {}, ready_after, set(fail)
        self.created, self.deleted = [], []

    def create(self, *, parent, body):
        name = f"{parent}/nodePools/{body['nodePool']['name']}"
        self.pools[name] = dict(body["nodePool"], status="PROVISIONING")
        self.reads[name] = 0
        self.created.append(body["nodePool"]["name"])

    def get(self, *, name):
        pool = self.pools.get(name)
        if pool is None:
            return None
        self.reads[name] += 1
        if pool["status"] == "PROVISIONING" and self.reads[name] > self.ready_after:
            pool["status"] = "ERROR" if pool["name"] in self.fail else "RUNNING"
        return pool

    def delete(self, *, name):
        self.deleted.append(name.rsplit("/", 1)[1])
        self.pools.pop(name, None)

    def list(self, *, parent):
        return [p for n, p in self.pools.items() if n.startswith(parent + "/")]


def _a4(**kw):
    return A4HighReplicatedJob.default_config().set(command="python -m axlearn_b200.common.launch_trainer_main --config x",
                                                    image="gcr.io/p/img:1", **kw)


def test_a4_replicated_job_manifest():
    fuse = GCSFuseMount(gcs_path="gs://bucket/runs/exp1")
    cfg = _a4(name="exp1", num_nodes=4, reservation="res-b200", priority_class="high", service_account="sa",
              gcsfuse_mount=fuse, mounts=[HostMount(name="data", mount_path="/data", host_path="/mnt/stateful/data"),
                                          EphemeralDiskMount(storage_class="hyperdisk-balanced", size_gb=500)],
              env_vars={"FOO": "1"}, disable_nvls=True, output_dir="/output/exp1")
    (entry,) = cfg.instantiate()()
    assert entry["name"] == "job" and entry["replicas"] == 1
    job = entry["template"]
    assert job["spec"]["parallelism"] == 4 and job["spec"]["completionMode"] == "Indexed" and job["spec"]["backoffLimit"] == 0
    assert job["metadata"]["annotations"]["alpha.jobset.sigs.k8s.io/exclusive-topology"] == "cloud.google.com/gke-nodepool"
    pod = job["spec"]["template"]
    assert pod["metadata"]["annotations"]["gke-gcsfuse/volumes"] == "true"
    spec = pod["spec"]
    assert spec["nodeSelector"] == {"cloud.google.com/gke-accelerator": "nvidia-b200",
                                    "node.kubernetes.io/instance-type": "a4-highgpu-8g",
                                    "cloud.google.com/reservation-name": "res-b200"}
    assert spec["restartPolicy"] == "Never" and spec["hostNetwork"] and spec["priorityClassName"] == "high"
    (container,) = spec["containers"]
    env = {e["name"]: e.get("value") for e in container["env"]}
    assert env["MASTER_ADDR"] == "exp1-job-0-0.exp1" and env["NUM_PROCESSES"] == "32" and env["FOO"] == "1"
    assert env["NCCL_IB_GID_INDEX"] == "3" and env["NCCL_NVLS_ENABLE"] == "0" and env["TORCH_SYMM_MEM_DISABLE_MULTICAST"] == "1"
    assert "NODE_RANK" in env and container["resources"]["limits"]["nvidia.com/gpu"] == "8"
    assert "--nnodes=4" in container["command"][2] and "-m axlearn_b200.common.launch_trainer_main" in container["command"][2]
    volumes = {v["name"]: v for v in spec["volumes"]}
    assert volumes["gcs-fuse-csi-ephemeral"]["csi"]["volumeAttributes"]["bucketName"] == "bucket"
    assert "only-dir=runs/exp1" in volumes["gcs-fuse-csi-ephemeral"]["csi"]["volumeAttributes"]["mountOptions"]
    assert volumes["data"]["hostPath"]["path"] == "/mnt/stateful/data" and "gib" in volumes
    assert volumes["persistent-disk"]["ephemeral"]["volumeClaimTemplate"]["spec"]["resources"]["requests"]["storage"] == "500Gi"
    mounts = {m["name"]: m["mountPath"] for m in container["volumeMounts"]}
    assert mounts["gcs-fuse-csi-ephemeral"] == "/output" and mounts["shared-memory"] == "/dev/shm"


def test_builder_validation_and_variants():
    with pytest.raises(ValueError):
        _a4(name="x", num_nodes=0).instantiate()
    with pytest.raises(ValueError):
        GPUReplicatedJob.default_config().set(name="x", command="c", image="i", machine_type="n1-standard").instantiate()
    with pytest.raises(ValueError):
        GCSFuseMount(gcs_path="bucket/x").volume()
    with pytest.raises(ValueError):
        JobDependency.default_config().set(name="a", status="Started").instantiate()
    ultra = A3UltraReplicatedJob.default_config().set(name="u", command="train.py", image="i", enable_spot=True).instantiate()
    pod = ultra()[0]["template"]["spec"]["template"]["spec"]
    assert pod["nodeSelector"]["cloud.google.com/gke-accelerator"] == "nvidia-h200-141gb"
    assert pod["nodeSelector"]["cloud.google.com/gke-spot"] == "true" and len(pod["tolerations"]) == 2
    assert "NCCL_NVLS_CHUNKSIZE" not in {e["name"] for e in pod["containers"][0]["env"]}
    assert "annotations" not in ultra()[0]["template"]["metadata"]      # single node: no exclusive topology

    class Bundler:
        def id(self, name):
            return f"registry/{name}:tag"

    no_image = A4HighReplicatedJob.default_config().set(name="b", command="c")
    assert no_image.instantiate(bundler=Bundler())()[0]["template"]["spec"]["template"]["spec"]["containers"][0]["image"] == "registry/b:tag"
    with pytest.raises(ValueError):
        no_image.instantiate()()


def test_composite_jobs_and_dependencies():
    workers = _a4(num_nodes=2, depends_on=[JobDependency.default_config().set(name="service", status="Ready")])
    service = A3UltraReplicatedJob.default_config().set(command="python serve.py", image="img")
    comp = CompositeReplicatedJob.default_config().set(inner={"service": service, "workers": workers})
    job = GKEJob.default_config().set(name="exp2", builder=comp, namespace="ml", max_restarts=3, queue="team-q")
    fake = FakeKubernetes()
    gke = job.instantiate(api=fake)
    body = gke.build_jobset()
    assert [r["name"] for r in body["spec"]["replicatedJobs"]] == ["service", "workers"]
    assert body["spec"]["replicatedJobs"][1]["dependsOn"] == [{"name": "service", "status": "Ready"}]
    assert body["spec"]["failurePolicy"] == {"maxRestarts": 3} and body["metadata"]["labels"]["kueue.x-k8s.io/queue-name"] == "team-q"
    # The coordinator address names the replicated job the pod belongs to.
    env = {e["name"]: e.get("value") for e in body["spec"]["replicatedJobs"][1]["template"]["spec"]["template"]["spec"]["containers"][0]["env"]}
    assert env["MASTER_ADDR"] == "exp2-workers-0-0.exp2"
    assert gke.status() == JobSetStatus.NOT_STARTED
    gke.execute()
    assert ("ml", "exp2") in fake.jobsets and gke.status() == JobSetStatus.PENDING
    fake.jobsets[("ml", "exp2")]["status"] = {"replicatedJobsStatus": [{"name": "service", "ready": 1}, {"name": "workers", "ready": 1}]}
    assert gke.status() == JobSetStatus.READY
    fake.jobsets[("ml", "exp2")]["status"] = {"restarts": 1, "replicatedJobsStatus": [{"name": "service", "ready": 1}]}
    assert gke.status() == JobSetStatus.RESCHEDULED
    fake.jobsets[("ml", "exp2")]["status"] = {"conditions": [{"type": "Failed", "status": "True"}]}
    assert gke.status() == JobSetStatus.FAILED
    assert jobset_status({"status": {"conditions": [{"type": "Completed", "status": "True"}]}}) == JobSetStatus.SUCCEEDED
    gke._delete()  # pylint: disable=protected-access
    assert gke.status() == JobSetStatus.NOT_STARTED


def test_node_pool_names_and_bodies():
    a = node_pool.construct_node_pool_name(jobset_namespace="ns", jobset_name="j" * 60, index=0)
    b = node_pool.construct_node_pool_name(jobset_namespace="ns", jobset_name="j" * 60, index=1)
    assert len(a) == 40 and a != b and a.startswith("j" * 34 + "-")
    body = node_pool.node_pool_body(name="p", zone="us-central1-b", num_nodes=4, machine_type="a4-highgpu-8g",
                                    accelerator="nvidia-b200", reservation="r", additional_labels={"k": "v"})
    np_ = body["nodePool"]
    assert np_["initialNodeCount"] == 4 and np_["placementPolicy"] == {"type": "COMPACT"}
    assert np_["config"]["accelerators"][0]["acceleratorCount"] == "8" and np_["config"]["labels"] == {"k": "v"}
    assert np_["config"]["reservationAffinity"]["values"] == ["r"] and "spot" not in np_["config"]
    with pytest.raises(node_pool.NodePoolValidationError):
        node_pool.node_pool_body(name="p", zone="z", num_nodes=1, machine_type="m", use_spot_vm=True, reservation="r")


def _provisioner(api, **kw):
    return GPUNodePoolProvisioner.default_config().set(
        project="proj", zone="us-central1-b", cluster="c1", name="prov", retry_interval=0, wait_timeout=5, **kw
    ).instantiate(api=api, sleep=lambda s: None)


def test_provisioner_creates_waits_and_deletes():
    api = FakeContainer(ready_after=2)
    job = GKEJob.default_config().set(name="exp3", builder=_a4(num_nodes=2, reservation="res")).instantiate(api=FakeKubernetes())
    prov = _provisioner(api, labels={"team": "ml"})
    (name,) = prov.create_for(job)
    pool = api.pools[f"projects/proj/locations/us-central1-b/clusters/c1/nodePools/{name}"]
    assert pool["status"] == "RUNNING" and pool["config"]["labels"]["job-name"] == "exp3"
    assert pool["config"]["labels"]["pre-provisioner-id"] == "prov" and pool["config"]["labels"]["team"] == "ml"
    prov.create_for(job)                       # idempotent: nothing is created twice
    assert api.created == [name]
    assert prov.orphaned(live_job_names=["exp3"]) == [] and prov.orphaned(live_job_names=[]) == [name]
    assert prov.delete_for(job) == [name] and api.deleted == [name] and not api.pools
    prov.delete_for(job)                       # deleting what is gone is fine
    # A pool that ends in ERROR raises.
    bad_api = FakeContainer(ready_after=1, fail=[name])
    with pytest.raises(node_pool.NodePoolCreationError):
        _provisioner(bad_api).create_for(job)
    # A pool that never becomes RUNNING times out.
    slow = FakeContainer(ready_after=10**9)
    with pytest.raises(node_pool.NodePoolCreationError):
        GPUNodePoolProvisioner.default_config().set(project="proj", zone="z", cluster="c", name="p", retry_interval=0,
                                                    wait_timeout=0.05).instantiate(api=slow, sleep=time.sleep).create_for(job)


def test_goodput_recorder_with_fake_client(tmp_path):
    from axlearn_b200.cloud.gcp.measurement import GoodputRecorder

    class Client:
        def __init__(self):
            self.events, self.reports = [], []

        def record(self, event, *, timestamp, **fields):
            self.events.append((event, fields))

        def upload(self, report):
            self.reports.append(report)

    client = Client()
    cfg = measurement.get_recorder_config("goodput", ["name=run1", "upload_interval=1"])
    cfg.rolling_window_size = (3600,)
    rec = cfg.instantiate(client=client)
    with rec.record_event(measurement.EventType.JOB):
        with rec.record_event(measurement.EventType.ACCELERATOR_INIT):
            time.sleep(0.01)
        for step in range(3):
            with rec.record_event(measurement.EventType.STEP, step):
                time.sleep(0.01)
    names = [e for e, _ in client.events]
    assert names[0] == "START_JOB" and names[-1] == "END_JOB" and names.count("START_STEP") == 3
    assert client.events[3][1]["step"] == 0
    report = rec.report()
    assert 0 < report["job"]["goodput"] <= 1 and report["job"]["badput"]["accelerator_init"] > 0
    assert report["window_3600s"]["productive_seconds"] == report["job"]["productive_seconds"]
    rec.stop_monitoring()
    assert client.reports and client.reports[-1]["job"]["goodput"] == pytest.approx(report["job"]["goodput"], rel=0.2)
    # Other processes record only their job start / end.
    other = cfg.instantiate(client=client, process_index=1)
    before = len(client.events)
    other.record(measurement.Event.START_STEP, 1)
    other.record(measurement.Event.START_JOB)
    assert len(client.events) == before + 1
    # Without a client the events go to a file under upload_dir.
    file_rec = measurement.get_recorder_config("goodput", ["name=run2", f"upload_dir={tmp_path}"]).instantiate()
    file_rec.record(measurement.Event.START_JOB)
    assert (tmp_path / "goodput_run2.jsonl").read_text().count("START_JOB") == 1


def test_settings_files_and_gcp_cli(tmp_path, monkeypatch, capsys):
    import json
    import os

    from axlearn_b200.cli import main as cli
    from axlearn_b200.cloud.common import config as settings

    root = tmp_path / "repo"
    (root / ".axlearn").mkdir(parents=True)
    (root / ".axlearn" / "axlearn.default.config").write_text(
        '[gcp]\n_active = "proj:us-central1-b"\n\n[gcp."proj:us-central1-b"]\nproject = "proj"\nzone = "us-central1-b"\n'
        'docker_image = "gcr.io/proj/img:1"\nreservation = "res-b200"\n\n[gcp."other:europe-west4-a"]\nproject = "other"\n'
        'zone = "europe-west4-a"\ndocker_image = "gcr.io/other/img:2"\n')
    monkeypatch.chdir(root)
    monkeypatch.setenv("HOME", str(tmp_path / "home"))
    path, gcp = settings.load_configs("gcp")
    assert path.endswith("axlearn.default.config") and gcp["_active"] == "proj:us-central1-b"
    assert settings.gcp_settings("docker_image") == "gcr.io/proj/img:1"
    assert settings.gcp_settings("env_id") == "us-central1-b"                       # falls back to the zone
    assert settings.gcp_settings("docker_image", project="other", env_id="europe-west4-a") == "gcr.io/other/img:2"
    assert settings.gcp_settings("missing", required=False) is None
    with pytest.raises(SystemExit):
        settings.gcp_settings("missing")
    # A user file overrides the default file key by key.
    user = settings.update_configs("gcp", {**gcp, "_active": "other:europe-west4-a"})
    assert user == str(root / ".axlearn" / ".axlearn.config")
    assert settings.gcp_settings("project") == "other"
    assert settings.load_configs("gcp")[1]["proj:us-central1-b"]["reservation"] == "res-b200"
    os.remove(user)
    # The command line builds the JobSet from those settings.
    assert cli.main(["gcp", "manifest", "--name", "run1", "--num_nodes", "2", "--output_dir", "gs://b/out",
                     "--fault_tolerant", "python", "-m", "train", "--x=1"]) == 0
    out = capsys.readouterr().out
    import yaml

    jobset = yaml.safe_load(out)
    pod = jobset["spec"]["replicatedJobs"][0]["template"]["spec"]["template"]["spec"]
    assert jobset["metadata"]["name"] == "run1" and pod["containers"][0]["image"] == "gcr.io/proj/img:1"
    assert pod["nodeSelector"]["cloud.google.com/reservation-name"] == "res-b200"
    assert "-m train --x=1" in pod["containers"][0]["command"][2]
    env = {e["name"]: e.get("value") for e in pod["containers"][0]["env"]}
    assert env["NCCL_NVLS_ENABLE"] == "0" and env["OUTPUT_DIR"] == "/output"
    assert cli.main(["gcp", "config", "--activate", "other:europe-west4-a"]) == 0
    assert settings.gcp_settings("project") == "other"
    assert cli.main(["gcp", "config"]) == 0
    assert json.loads(capsys.readouterr().out.split("\n", 1)[1])["gcp"]["_active"] == "other:europe-west4-a"
