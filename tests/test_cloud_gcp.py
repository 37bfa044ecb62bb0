"""JobSet manifests for B200 node pools; lifecycle event queue."""
import threading

import pytest

from axlearn_b200.cloud.common.event_queue import FileQueueClient, InMemoryQueueClient, JobLifecycleEvent
from axlearn_b200.cloud.gcp.jobset import A4_HIGH_NCCL_ENV, GPUJobSet


def _job(**kw):
    kw.setdefault("num_nodes", 4)
    return GPUJobSet.default_config().set(
        name="fuji70b", image="registry/train:1",
        command="python -m axlearn_b200.common.launch_trainer_main --module=text.gpt.c4_trainer --config=fuji-70B-v2-flash",
        **kw).instantiate()


def test_a4_high_manifest():
    m = _job(env_vars={"NCCL_DEBUG": "INFO"}, output_claim="ckpt", output_dir="/ckpt", reservation="r1", max_restarts=3).build()
    assert m["kind"] == "JobSet" and m["spec"]["failurePolicy"] == {"maxRestarts": 3}
    job = m["spec"]["replicatedJobs"][0]["template"]
    assert job["spec"]["parallelism"] == 4 and job["spec"]["completionMode"] == "Indexed"
    pod = job["spec"]["template"]["spec"]
    assert pod["nodeSelector"]["cloud.google.com/gke-accelerator"] == "nvidia-b200"
    assert pod["nodeSelector"]["cloud.google.com/reservation-name"] == "r1"
    c = pod["containers"][0]
    assert c["resources"]["limits"] == {"nvidia.com/gpu": "8"}
    env = {e["name"]: e.get("value") for e in c["env"]}
    assert env["NCCL_IB_GID_INDEX"] == A4_HIGH_NCCL_ENV["NCCL_IB_GID_INDEX"] and env["NCCL_DEBUG"] == "INFO"
    assert env["MASTER_ADDR"] == "fuji70b-workers-0-0.fuji70b" and env["NUM_NODES"] == "4"
    rank = [e for e in c["env"] if e["name"] == "NODE_RANK"][0]
    assert "job-completion-index" in rank["valueFrom"]["fieldRef"]["fieldPath"]
    cmd = c["command"][-1]
    assert "--nnodes=4 --nproc-per-node=8 --node-rank=$NODE_RANK" in cmd and cmd.endswith("--config=fuji-70B-v2-flash")
    assert "-m axlearn_b200.common.launch_trainer_main" in cmd and "run python" not in cmd
    assert {"name": "gib", "mountPath": "/usr/local/gib"} in c["volumeMounts"]
    assert {"name": "output", "mountPath": "/ckpt"} in c["volumeMounts"]
    assert any(v.get("persistentVolumeClaim") == {"claimName": "ckpt"} for v in pod["volumes"])
    assert "exclusive-topology" in str(job["metadata"])


def test_yaml_round_trip_and_other_machine_types():
    yaml = pytest.importorskip("yaml")
    job = _job(machine_type="a3-ultragpu-8g", num_nodes=1)
    m = yaml.safe_load(job.to_yaml())
    pod = m["spec"]["replicatedJobs"][0]["template"]["spec"]["template"]["spec"]
    assert pod["nodeSelector"]["cloud.google.com/gke-accelerator"] == "nvidia-h200-141gb"
    assert not any(v["name"] == "gib" for v in pod["volumes"])
    assert job.submit_command("/tmp/j.yaml")[:2] == ["kubectl", "apply"]
    with pytest.raises(ValueError):
        _job(machine_type="tpu-v5").build()


def test_event_queue_clients(tmp_path):
    mem = InMemoryQueueClient()
    mem.publish(JobLifecycleEvent("j1", "ACTIVE"))
    assert mem.events[0].state == "ACTIVE"
    q = FileQueueClient(str(tmp_path / "events" / "log.jsonl"))
    threads = [threading.Thread(target=lambda i=i: [q.publish(JobLifecycleEvent(f"job{i}", "PENDING", details="x" * 200))
                                                   for _ in range(50)]) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    events = q.read_all()
    assert len(events) == 200 and q.dropped == 0 and all(e["timestamp"] > 0 for e in events)
