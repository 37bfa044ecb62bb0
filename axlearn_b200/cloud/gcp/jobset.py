"""Kubernetes JobSet manifests for multi-node B200 (GKE ``a4-highgpu-8g``) training jobs.

Counterpart of the GPU replicated-job builders in axlearn/cloud/gcp/jobset_utils.py
(``GPUReplicatedJob`` and ``A4HighReplicatedJob`` :1800-1900) and of the JobSet wrapper in
axlearn/cloud/gcp/job.py.  A job is ``num_nodes`` pods of 8 GPUs; every pod runs one launcher that
starts one process per GPU (``torch.distributed.run``) and rendezvouses at pod 0 through the
JobSet's headless service.  Only the manifest is built here: it is plain data, applied with
``kubectl apply -f`` (``to_yaml``) or through any Kubernetes client.

The network settings are the ones published for A4 (B200 with RoCE / gIB) node pools: the NCCL
gIB plugin mounted from the host, GID index 3, adaptive routing, traffic classes 52 / 84, and NVLS
chunk sizes for the in-node NVSwitch.
"""

from __future__ import annotations

import shlex
from typing import Any, Optional, Sequence

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class

GPUS_PER_NODE = 8
_ACCELERATOR = {"a4-highgpu-8g": "nvidia-b200", "a3-ultragpu-8g": "nvidia-h200-141gb", "a3-megagpu-8g": "nvidia-h100-mega-80gb"}

A4_HIGH_NCCL_ENV = {
    "LD_LIBRARY_PATH": "/usr/local/gib/lib64:/usr/local/nvidia/lib64",
    "CUDA_DEVICE_MAX_CONNECTIONS": "1",
    "NCCL_DEBUG": "WARN",
    "NCCL_CROSS_NIC": "0",
    "NCCL_NET_GDR_LEVEL": "PIX",
    "NCCL_P2P_NET_CHUNKSIZE": "131072",
    "NCCL_P2P_PCI_CHUNKSIZE": "131072",
    "NCCL_P2P_NVL_CHUNKSIZE": "524288",
    "NCCL_NVLS_CHUNKSIZE": "524288",
    "NCCL_IB_GID_INDEX": "3",
    "NCCL_IB_ADAPTIVE_ROUTING": "1",
    "NCCL_IB_QPS_PER_CONNECTION": "4",
    "NCCL_IB_TC": "52",
    "NCCL_IB_FIFO_TC": "84",
}


class GPUJobSet(Configurable):
    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED
        image: Required[str] = REQUIRED
        command: Required[str] = REQUIRED                 # what every process runs, e.g. "python -m ... --flags"
        num_nodes: int = 1
        machine_type: str = "a4-highgpu-8g"
        namespace: str = "default"
        env_vars: dict = {}
        max_restarts: int = 0                              # whole-JobSet restarts on failure
        output_dir: Optional[str] = None                   # a shared volume path mounted at /output
        output_claim: Optional[str] = None                 # PersistentVolumeClaim backing it
        service_account: Optional[str] = None
        priority_class: Optional[str] = None
        reservation: Optional[str] = None
        rendezvous_port: int = 29500
        termination_grace_period_seconds: int = 60
        launcher: str = "python -m torch.distributed.run"
        extra_node_selector: dict = {}
        tolerations: Sequence[dict] = ({"key": "nvidia.com/gpu", "operator": "Exists", "effect": "NoSchedule"},)

    # ------------------------------------------------------------------ pieces
    def _coordinator(self) -> str:
        cfg = self.config
        # <jobset>-<replicated job>-<job index>-<pod index>.<jobset>: the JobSet's headless service.
        return f"{cfg.name}-workers-0-0.{cfg.name}"

    def _env(self) -> list[dict]:
        cfg = self.config
        env = dict(A4_HIGH_NCCL_ENV) if cfg.machine_type == "a4-highgpu-8g" else {"NCCL_DEBUG": "WARN"}
        env.update({"MASTER_ADDR": self._coordinator(), "MASTER_PORT": str(cfg.rendezvous_port),
                    "NUM_NODES": str(cfg.num_nodes), "GPUS_PER_NODE": str(GPUS_PER_NODE)})
        env.update({k: str(v) for k, v in cfg.env_vars.items()})
        out = [{"name": k, "value": v} for k, v in env.items()]
        out.append({"name": "NODE_RANK", "valueFrom": {"fieldRef": {
            "fieldPath": "metadata.annotations['batch.kubernetes.io/job-completion-index']"}}})
        return out

    def _command(self) -> list[str]:
        cfg = self.config
        launch = (f"{cfg.launcher} --nnodes={cfg.num_nodes} --nproc-per-node={GPUS_PER_NODE} "
                  f"--node-rank=$NODE_RANK --master-addr=$MASTER_ADDR --master-port=$MASTER_PORT")
        program = cfg.command.strip()
        if program.startswith("python "):
            program = program[len("python "):]
        return ["bash", "-c", f"exec {launch} {program}"]

    def _container(self) -> dict:
        cfg = self.config
        mounts = [{"name": "shared-memory", "mountPath": "/dev/shm"}, {"name": "nvidia", "mountPath": "/usr/local/nvidia"}]
        if cfg.machine_type == "a4-highgpu-8g":
            mounts.append({"name": "gib", "mountPath": "/usr/local/gib"})
        if cfg.output_claim:
            mounts.append({"name": "output", "mountPath": cfg.output_dir or "/output"})
        return dict(name=cfg.name, image=cfg.image, command=self._command(), env=self._env(),
                    ports=[{"containerPort": cfg.rendezvous_port}], securityContext={"privileged": True},
                    resources={"limits": {"nvidia.com/gpu": str(GPUS_PER_NODE)}}, volumeMounts=mounts)

    def _volumes(self) -> list[dict]:
        cfg = self.config
        vols = [{"name": "shared-memory", "emptyDir": {"medium": "Memory"}},
                {"name": "nvidia", "hostPath": {"path": "/home/kubernetes/bin/nvidia"}}]
        if cfg.machine_type == "a4-highgpu-8g":
            vols.append({"name": "gib", "hostPath": {"path": "/home/kubernetes/bin/gib"}})
        if cfg.output_claim:
            vols.append({"name": "output", "persistentVolumeClaim": {"claimName": cfg.output_claim}})
        return vols

    def _pod_spec(self) -> dict:
        cfg = self.config
        if cfg.machine_type not in _ACCELERATOR:
            raise ValueError(f"unknown machine type {cfg.machine_type}; known: {sorted(_ACCELERATOR)}")
        selector = {"cloud.google.com/gke-accelerator": _ACCELERATOR[cfg.machine_type],
                    "node.kubernetes.io/instance-type": cfg.machine_type, **cfg.extra_node_selector}
        if cfg.reservation:
            selector["cloud.google.com/reservation-name"] = cfg.reservation
        spec: dict[str, Any] = dict(
            restartPolicy="Never", hostNetwork=True, dnsPolicy="ClusterFirstWithHostNet",
            terminationGracePeriodSeconds=cfg.termination_grace_period_seconds, nodeSelector=selector,
            tolerations=[dict(t) for t in cfg.tolerations], containers=[self._container()], volumes=self._volumes())
        if cfg.service_account:
            spec["serviceAccountName"] = cfg.service_account
        if cfg.priority_class:
            spec["priorityClassName"] = cfg.priority_class
        return spec

    # ------------------------------------------------------------------ manifest
    def build(self) -> dict:
        cfg = self.config
        if cfg.num_nodes < 1:
            raise ValueError("num_nodes must be positive")
        job = dict(
            metadata={"annotations": {"alpha.jobset.sigs.k8s.io/exclusive-topology": "cloud.google.com/gke-nodepool"}}
            if cfg.num_nodes > 1 else {},
            spec=dict(parallelism=cfg.num_nodes, completions=cfg.num_nodes, completionMode="Indexed", backoffLimit=0,
                      template=dict(metadata={"labels": {"app": cfg.name}}, spec=self._pod_spec())))
        return dict(
            apiVersion="jobset.x-k8s.io/v1alpha2", kind="JobSet",
            metadata=dict(name=cfg.name, namespace=cfg.namespace),
            spec=dict(failurePolicy={"maxRestarts": cfg.max_restarts},
                      network={"enableDNSHostnames": True, "subdomain": cfg.name},
                      replicatedJobs=[dict(name="workers", replicas=1, template=job)]))

    def to_yaml(self) -> str:
        import yaml  # pylint: disable=import-outside-toplevel

        return yaml.safe_dump(self.build(), sort_keys=False)

    def submit_command(self, manifest_path: str) -> list[str]:
        return ["kubectl", "apply", "-n", self.config.namespace, "-f", manifest_path]

    def delete_command(self) -> list[str]:
        return ["kubectl", "delete", "jobset", self.config.name, "-n", self.config.namespace, "--ignore-not-found"]
