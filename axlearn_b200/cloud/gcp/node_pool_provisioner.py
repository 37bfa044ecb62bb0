"""Creates and deletes the node pools a GKE GPU job runs on.

Parity target: axlearn/cloud/gcp/node_pool_provisioner.py (``NodePoolProvisioner`` :39 with
``create_for`` / ``delete_for``; the TPU provisioner :134-420 creates one pool per slice).  For GPU
jobs one pool holds all nodes of a replicated job (the JobSet pins a job to one pool with the
exclusive-topology annotation), so there is one pool per replicated job.
"""

from __future__ import annotations

import time
from typing import Callable, Optional

from axlearn_b200.cloud.gcp import node_pool
from axlearn_b200.cloud.gcp.job import GKEJob
from axlearn_b200.cloud.gcp.jobset_utils import ACCELERATOR_LABELS, GPUReplicatedJob
from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class

PRE_PROVISIONER_LABEL = "pre-provisioner-id"


class NodePoolProvisioner(Configurable):
    @config_class
    class Config(Configurable.Config):
        project: Required[str] = REQUIRED
        zone: Required[str] = REQUIRED
        cluster: Required[str] = REQUIRED
        name: Required[str] = REQUIRED
        service_account_email: Optional[str] = None
        retry_interval: int = 30
        wait_timeout: int = 30 * 60
        labels: Optional[dict] = None
        disk_type: Optional[str] = None

    def __init__(self, cfg, *, api: node_pool.ContainerApi, sleep: Callable[[float], None] = time.sleep):
        super().__init__(cfg)
        self._api = api
        self._sleep = sleep

    def create_for(self, job: GKEJob):
        raise NotImplementedError(type(self))

    def delete_for(self, job: GKEJob):
        raise NotImplementedError(type(self))


class GPUNodePoolProvisioner(NodePoolProvisioner):
    def _pools_for(self, job: GKEJob) -> list:
        """``(pool name, builder)`` for every GPU replicated job of the JobSet."""
        builder = job.builder
        inner = getattr(builder, "_inner", None)
        builders = list(inner.values()) if inner else [builder]
        gpu = [b for b in builders if isinstance(b, GPUReplicatedJob)]
        return [(node_pool.construct_node_pool_name(jobset_namespace=job.config.namespace, jobset_name=job.config.name,
                                                    index=i), b) for i, b in enumerate(gpu)]

    def create_for(self, job: GKEJob):
        cfg = self._config
        bodies = []
        for name, b in self._pools_for(job):
            bcfg = b.config
            machine = bcfg.machine_type or b.MACHINE_TYPE
            bodies.append(node_pool.node_pool_body(
                name=name, zone=cfg.zone, num_nodes=bcfg.num_nodes, machine_type=machine,
                accelerator=ACCELERATOR_LABELS[machine], use_spot_vm=True if bcfg.enable_spot else None,
                reservation=bcfg.reservation, disk_type=cfg.disk_type, service_account_email=cfg.service_account_email,
                additional_labels={**(cfg.labels or {}), "provisioner-nodepool-id": name, "job-name": job.config.name},
                pre_provisioner_id=cfg.name))
        node_pool.create_node_pools(self._api, project=cfg.project, zone=cfg.zone, cluster=cfg.cluster, bodies=bodies,
                                    wait_timeout=cfg.wait_timeout, retry_interval=cfg.retry_interval, sleep=self._sleep)
        return [b["nodePool"]["name"] for b in bodies]

    def delete_for(self, job: GKEJob):
        cfg = self._config
        names = [n for n, _ in self._pools_for(job)]
        node_pool.delete_node_pools(self._api, project=cfg.project, zone=cfg.zone, cluster=cfg.cluster, names=names,
                                    wait_timeout=cfg.wait_timeout, retry_interval=cfg.retry_interval, sleep=self._sleep)
        return names

    def orphaned(self, live_job_names) -> list:
        """Pools made by this provisioner whose job is not among ``live_job_names``."""
        cfg = self._config
        mine = node_pool.list_node_pools_by_label_key(self._api, project=cfg.project, zone=cfg.zone, cluster=cfg.cluster,
                                                      label_key=PRE_PROVISIONER_LABEL).get(cfg.name, [])
        live = set(live_job_names)
        return [p["name"] for p in mine if p.get("config", {}).get("labels", {}).get("job-name") not in live]
