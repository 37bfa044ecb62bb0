"""Replicated-job builders for Kubernetes JobSets on GKE GPU node pools.

Parity target: axlearn/cloud/gcp/jobset_utils.py -- ``VolumeMount`` / ``GCSFuseMount`` /
``HostMount`` / ``EphemeralDiskMount`` :72-140, ``BaseReplicatedJob`` :178, ``CompositeReplicatedJob``
:255, ``JobDependency`` :293, ``GPUReplicatedJob`` :1143 and the per-machine builders
(``A3UltraReplicatedJob`` :1696, ``A4HighReplicatedJob`` :1800).  The TPU and Pathways builders have
no counterpart here.

A builder turns a config into the ``replicatedJobs`` entries of a JobSet (plain nested dicts); the
JobSet itself is assembled and applied by ``cloud/gcp/job.py``.  A worker pod runs one launcher
that starts one process per GPU (``torch.distributed.run``) and rendezvouses at pod 0 of the first
replicated job through the JobSet's headless service.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Optional, Sequence

from axlearn_b200.cloud.gcp.jobset import A4_HIGH_NCCL_ENV, GPUS_PER_NODE
from axlearn_b200.common import runtime_options
from axlearn_b200.common.config import REQUIRED, Configurable, InstantiableConfig, Required, config_class

# Machine type -> GKE accelerator label.
ACCELERATOR_LABELS = {
    "a4-highgpu-8g": "nvidia-b200",
    "a3-ultragpu-8g": "nvidia-h200-141gb",
    "a3-megagpu-8g": "nvidia-h100-mega-80gb",
    "a3-highgpu-8g": "nvidia-h100-80gb",
}

A3_ULTRA_NCCL_ENV = {
    "LD_LIBRARY_PATH": "/usr/local/gib/lib64:/usr/local/nvidia/lib64",
    "NCCL_DEBUG": "WARN",
    "NCCL_CROSS_NIC": "0",
    "NCCL_NET_GDR_LEVEL": "PIX",
    "NCCL_P2P_NET_CHUNKSIZE": "131072",
    "NCCL_IB_GID_INDEX": "3",
    "NCCL_IB_ADAPTIVE_ROUTING": "1",
    "NCCL_IB_QPS_PER_CONNECTION": "4",
    "NCCL_IB_TC": "52",
    "NCCL_IB_FIFO_TC": "84",
}


@dataclasses.dataclass(kw_only=True)
class VolumeMount:
    name: str
    mount_path: str
    read_only: bool = False

    def volume(self) -> dict:
        raise NotImplementedError(type(self))

    def mount(self) -> dict:
        return {"name": self.name, "mountPath": self.mount_path, "readOnly": self.read_only}


@dataclasses.dataclass(kw_only=True)
class GCSFuseMount(VolumeMount):
    """A bucket path mounted through the Cloud Storage FUSE CSI driver (an ephemeral volume; the
    driver's sidecar is requested with pod annotations, see ``pod_annotations``)."""

    gcs_path: str
    name: str = "gcs-fuse-csi-ephemeral"
    mount_path: str = "/output"
    cpu: str = "250m"
    memory: str = "256Mi"
    ephemeral_gb: str = "5Gi"
    http_client_timeout: str = "0s"

    def _bucket_and_dir(self) -> tuple:
        if not self.gcs_path.startswith("gs://"):
            raise ValueError(f"gcs_path must start with gs://: {self.gcs_path}")
        bucket, _, sub = self.gcs_path[len("gs://"):].partition("/")
        return bucket, sub.rstrip("/")

    def volume(self) -> dict:
        bucket, sub = self._bucket_and_dir()
        options = ["implicit-dirs", f"http-client-timeout={self.http_client_timeout}"]
        if sub:
            options.append(f"only-dir={sub}")
        return {"name": self.name, "csi": {"driver": "gcsfuse.csi.storage.gke.io", "readOnly": self.read_only,
                                          "volumeAttributes": {"bucketName": bucket, "mountOptions": ",".join(options)}}}

    def pod_annotations(self) -> dict:
        return {"gke-gcsfuse/volumes": "true", "gke-gcsfuse/cpu-request": self.cpu,
                "gke-gcsfuse/memory-request": self.memory, "gke-gcsfuse/ephemeral-storage-request": self.ephemeral_gb,
                "gke-gcsfuse/cpu-limit": "0", "gke-gcsfuse/memory-limit": "0", "gke-gcsfuse/ephemeral-storage-limit": "0"}


@dataclasses.dataclass(kw_only=True)
class HostMount(VolumeMount):
    host_path: str
    type: str = "Directory"

    def volume(self) -> dict:
        return {"name": self.name, "hostPath": {"path": self.host_path, "type": self.type}}


@dataclasses.dataclass(kw_only=True)
class EphemeralDiskMount(VolumeMount):
    """A per-pod PersistentVolumeClaim created with the pod and deleted with it."""

    storage_class: str
    size_gb: int
    name: str = "persistent-disk"
    mount_path: str = "/mnt"

    def volume(self) -> dict:
        return {"name": self.name, "ephemeral": {"volumeClaimTemplate": {"spec": {
            "accessModes": ["ReadWriteOnce"], "storageClassName": self.storage_class,
            "resources": {"requests": {"storage": f"{self.size_gb}Gi"}}}}}}


class JobDependency(Configurable):
    """``dependsOn`` entry: start this replicated job when ``name`` is ``status`` (Ready / Complete)."""

    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED
        status: str = "Ready"

    def __init__(self, cfg):
        super().__init__(cfg)
        if cfg.status not in ("Ready", "Complete"):
            raise ValueError(f"status must be Ready or Complete, got {cfg.status}")

    def build_depends_on(self) -> dict:
        return {"name": self._config.name, "status": self._config.status}


class BaseReplicatedJob(Configurable):
    """Builds ``replicatedJobs`` entries."""

    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED            # the JobSet's name
        job_name: str = "job"                     # this replicated job's name inside the JobSet
        image: Optional[str] = None               # container image (None: the bundler's id for `name`)
        command: Required[str] = REQUIRED
        env_vars: dict = {}
        service_account: Optional[str] = None
        output_dir: Optional[str] = None
        depends_on: Sequence[InstantiableConfig] = ()

    def __init__(self, cfg, *, bundler: Any = None):
        super().__init__(cfg)
        self._bundler = bundler
        self._depends_on = [d.instantiate() for d in cfg.depends_on]

    def __call__(self) -> Sequence[dict]:
        raise NotImplementedError(type(self))

    def get_workload_labels(self) -> dict:
        return {}

    def get_workload_annotations(self) -> dict:
        return {}

    def _image(self) -> str:
        cfg = self._config
        if cfg.image:
            return cfg.image
        if self._bundler is None:
            raise ValueError("either `image` or a bundler is needed")
        return self._bundler.id(cfg.name)


class CompositeReplicatedJob(BaseReplicatedJob):
    """Several builders in one JobSet (e.g. workers plus a sidecar service)."""

    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED   # the JobSet's name, handed to every inner builder
        inner: dict = {}                 # job_name -> builder config

    def __init__(self, cfg, *, bundler: Any = None):
        Configurable.__init__(self, cfg)  # pylint: disable=non-parent-init-called
        if not cfg.inner:
            raise ValueError("CompositeReplicatedJob needs at least one inner builder")
        self._inner = {job_name: c.clone(name=cfg.name, job_name=job_name).instantiate(bundler=bundler)
                       for job_name, c in cfg.inner.items()}

    def __call__(self) -> Sequence[dict]:
        out = []
        for builder in self._inner.values():
            out.extend(builder())
        names = [e["name"] for e in out]
        if len(set(names)) != len(names):
            raise ValueError(f"replicated job names must be unique: {names}")
        return out

    def get_workload_labels(self) -> dict:
        labels = {}
        for b in self._inner.values():
            labels.update(b.get_workload_labels())
        return labels

    def get_workload_annotations(self) -> dict:
        ann = {}
        for b in self._inner.values():
            ann.update(b.get_workload_annotations())
        return ann


class GPUReplicatedJob(BaseReplicatedJob):
    """``num_nodes`` pods of eight GPUs each: the parts common to every GPU machine type."""

    MACHINE_TYPE: Optional[str] = None
    NCCL_ENV: dict = {"NCCL_DEBUG": "WARN"}

    @config_class
    class Config(BaseReplicatedJob.Config):
        num_nodes: int = 1
        machine_type: Optional[str] = None
        reservation: Optional[str] = None
        priority_class: Optional[str] = None
        enable_spot: bool = False
        rendezvous_port: int = 29500
        launcher: str = "python -m torch.distributed.run"
        mounts: Sequence[VolumeMount] = ()
        gcsfuse_mount: Optional[GCSFuseMount] = None
        termination_grace_period_seconds: int = 60
        # FT-supervised jobs must not bind ranks to NVLink multicast objects.
        disable_nvls: bool = False

    def __init__(self, cfg, *, bundler: Any = None):
        super().__init__(cfg, bundler=bundler)
        if cfg.num_nodes < 1:
            raise ValueError("num_nodes must be positive")
        self._machine_type = cfg.machine_type or self.MACHINE_TYPE
        if self._machine_type not in ACCELERATOR_LABELS:
            raise ValueError(f"unknown machine type {self._machine_type}; known: {sorted(ACCELERATOR_LABELS)}")

    # ------------------------------------------------------------------ pieces
    def _coordinator(self) -> str:
        cfg = self._config
        return f"{cfg.name}-{cfg.job_name}-0-0.{cfg.name}"

    def _env(self) -> list:
        cfg = self._config
        # Framework defaults for this topology first; the fabric's NCCL settings and the user's
        # own variables override them.
        env = runtime_options.env_from_options(runtime_options.default_runtime_options(
            instance_type="b200", num_gpus=GPUS_PER_NODE, num_nodes=cfg.num_nodes))
        env.update(self.NCCL_ENV)
        env.update({"MASTER_ADDR": self._coordinator(), "MASTER_PORT": str(cfg.rendezvous_port),
                    "NUM_NODES": str(cfg.num_nodes), "GPUS_PER_NODE": str(GPUS_PER_NODE),
                    "NUM_PROCESSES": str(cfg.num_nodes * GPUS_PER_NODE)})
        if cfg.disable_nvls:
            env.update({"NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1"})
        if cfg.output_dir:
            env["OUTPUT_DIR"] = cfg.output_dir
        env.update({k: str(v) for k, v in cfg.env_vars.items()})
        out = [{"name": k, "value": v} for k, v in env.items()]
        out.append({"name": "NODE_RANK", "valueFrom": {"fieldRef": {
            "fieldPath": "metadata.annotations['batch.kubernetes.io/job-completion-index']"}}})
        return out

    def _command(self) -> list:
        cfg = self._config
        launch = (f"{cfg.launcher} --nnodes={cfg.num_nodes} --nproc-per-node={GPUS_PER_NODE} "
                  f"--node-rank=$NODE_RANK --master-addr=$MASTER_ADDR --master-port=$MASTER_PORT")
        program = cfg.command.strip()
        if program.startswith("python "):
            program = program[len("python "):]
        return ["bash", "-c", f"exec {launch} {program}"]

    def _all_mounts(self) -> list:
        cfg = self._config
        mounts = list(cfg.mounts)
        if cfg.gcsfuse_mount is not None:
            mounts.append(cfg.gcsfuse_mount)
        return mounts

    def _machine_volumes(self) -> list:
        """``(volume, mount)`` pairs every pod of this machine type needs."""
        return [({"name": "shared-memory", "emptyDir": {"medium": "Memory"}},
                 {"name": "shared-memory", "mountPath": "/dev/shm"}),
                ({"name": "nvidia-install-dir-host", "hostPath": {"path": "/home/kubernetes/bin/nvidia/lib64"}},
                 {"name": "nvidia-install-dir-host", "mountPath": "/usr/local/nvidia/lib64"})]

    def _build_init_containers(self) -> list:
        return []

    def _build_main_container(self) -> dict:
        cfg = self._config
        mounts = [m for _, m in self._machine_volumes()] + [m.mount() for m in self._all_mounts()]
        return dict(name=cfg.name, image=self._image(), command=self._command(), env=self._env(),
                    ports=[{"containerPort": cfg.rendezvous_port}], securityContext={"privileged": True},
                    resources={"limits": {"nvidia.com/gpu": str(GPUS_PER_NODE)}}, volumeMounts=mounts)

    def _build_pod(self) -> dict:
        cfg = self._config
        selector = {"cloud.google.com/gke-accelerator": ACCELERATOR_LABELS[self._machine_type],
                    "node.kubernetes.io/instance-type": self._machine_type}
        if cfg.reservation:
            selector["cloud.google.com/reservation-name"] = cfg.reservation
        if cfg.enable_spot:
            selector["cloud.google.com/gke-spot"] = "true"
        tolerations = [{"key": "nvidia.com/gpu", "operator": "Exists", "effect": "NoSchedule"}]
        if cfg.enable_spot:
            tolerations.append({"key": "cloud.google.com/gke-spot", "operator": "Equal", "value": "true",
                                "effect": "NoSchedule"})
        annotations = {"kubectl.kubernetes.io/default-container": cfg.name}
        if cfg.gcsfuse_mount is not None:
            annotations.update(cfg.gcsfuse_mount.pod_annotations())
        spec: dict = dict(
            terminationGracePeriodSeconds=cfg.termination_grace_period_seconds,
            restartPolicy="Never",           # a failed pod fails the Job; retries happen at JobSet level
            initContainers=self._build_init_containers(), hostNetwork=True, dnsPolicy="ClusterFirstWithHostNet",
            nodeSelector=selector, tolerations=tolerations, containers=[self._build_main_container()],
            volumes=[v for v, _ in self._machine_volumes()] + [m.volume() for m in self._all_mounts()])
        if cfg.service_account:
            spec["serviceAccountName"] = cfg.service_account
        if cfg.priority_class:
            spec["priorityClassName"] = cfg.priority_class
        return dict(metadata=dict(annotations=annotations, labels={"app": cfg.name, **self.get_workload_labels()}),
                    spec=spec)

    def __call__(self) -> Sequence[dict]:
        cfg = self._config
        metadata = {}
        if cfg.num_nodes > 1:
            # All pods of this job in one node pool (one network fabric).
            metadata["annotations"] = {"alpha.jobset.sigs.k8s.io/exclusive-topology": "cloud.google.com/gke-nodepool"}
        job = dict(metadata=metadata, spec=dict(
            parallelism=cfg.num_nodes, completions=cfg.num_nodes, completionMode="Indexed", backoffLimit=0,
            template=self._build_pod()))
        entry: dict = dict(name=cfg.job_name, replicas=1, template=job)
        if self._depends_on:
            entry["dependsOn"] = [d.build_depends_on() for d in self._depends_on]
        return [entry]

    def get_workload_labels(self) -> dict:
        return {"axlearn-b200/machine-type": self._machine_type}


class A4HighReplicatedJob(GPUReplicatedJob):
    """B200 nodes (``a4-highgpu-8g``): RoCE NICs driven by the gIB NCCL plugin mounted from the host."""

    MACHINE_TYPE = "a4-highgpu-8g"
    NCCL_ENV = A4_HIGH_NCCL_ENV

    def _machine_volumes(self) -> list:
        return super()._machine_volumes() + [
            ({"name": "gib", "hostPath": {"path": "/home/kubernetes/bin/gib"}}, {"name": "gib", "mountPath": "/usr/local/gib"})]


class A3UltraReplicatedJob(GPUReplicatedJob):
    """H200 nodes (``a3-ultragpu-8g``): the same RoCE / gIB arrangement without the NVLS chunk sizes."""

    MACHINE_TYPE = "a3-ultragpu-8g"
    NCCL_ENV = A3_ULTRA_NCCL_ENV

    def _machine_volumes(self) -> list:
        return super()._machine_volumes() + [
            ({"name": "gib", "hostPath": {"path": "/home/kubernetes/bin/gib"}}, {"name": "gib", "mountPath": "/usr/local/gib"})]
