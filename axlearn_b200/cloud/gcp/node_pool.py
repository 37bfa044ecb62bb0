"""GKE node pools for GPU jobs: request bodies and create / delete / list / status calls.

Parity target: axlearn/cloud/gcp/node_pool.py (``_node_pool_body`` :68, ``create_node_pool(s)``
:408-626, ``delete_node_pool(s)`` :281-406, ``list_node_pools_by_label_key`` :628,
``get_node_pool_status`` :665, ``construct_node_pool_name`` :709), for GPU machine types instead of
TPU slices.  The GKE container API is an interface (``ContainerApi``: the four REST calls of
``projects.locations.clusters.nodePools``); production code passes a client built on the
googleapiclient discovery document, tests pass a fake.
"""

from __future__ import annotations

import enum
import hashlib
import time
from typing import Any, Callable, Optional, Protocol, Sequence


class NodePoolCreationError(RuntimeError):
    pass


class NodePoolValidationError(RuntimeError):
    pass


class NodePoolDeletionError(RuntimeError):
    pass


class NodePoolStatus(enum.Enum):
    STATUS_UNSPECIFIED = "STATUS_UNSPECIFIED"
    PROVISIONING = "PROVISIONING"
    RUNNING = "RUNNING"
    RUNNING_WITH_ERROR = "RUNNING_WITH_ERROR"
    RECONCILING = "RECONCILING"
    STOPPING = "STOPPING"
    ERROR = "ERROR"
    NOT_EXIST = "NOT_EXIST"
    UNKNOWN = "UNKNOWN"


class ContainerApi(Protocol):
    """``parent`` = ``projects/P/locations/Z/clusters/C``; ``name`` = ``parent/nodePools/N``."""

    def create(self, *, parent: str, body: dict) -> Any: ...

    def get(self, *, name: str) -> Optional[dict]: ...       # None when the pool does not exist

    def delete(self, *, name: str) -> Any: ...

    def list(self, *, parent: str) -> Sequence[dict]: ...


def node_pool_parent(*, project: str, zone: str, cluster: str) -> str:
    return f"projects/{project}/locations/{zone}/clusters/{cluster}"


def node_pool_canonical_id(*, project: str, zone: str, cluster: str, name: str) -> str:
    return f"{node_pool_parent(project=project, zone=zone, cluster=cluster)}/nodePools/{name}"


def construct_node_pool_name(*, jobset_namespace: str, jobset_name: str, index: int) -> str:
    """At most 40 characters and unique per (namespace, JobSet, index): the first 34 characters of the
    JobSet's name, a dash, and 5 hex digits of a hash of ``namespace/name-index``."""
    digest = hashlib.md5(f"{jobset_namespace}/{jobset_name}-{index}".encode("utf-8")).hexdigest()
    return f"{jobset_name[:34]}-{digest[:5]}"


def node_pool_body(*, name: str, zone: str, num_nodes: int, machine_type: str, accelerator: Optional[str] = None,
                   gpus_per_node: int = 8, use_spot_vm: Optional[bool] = None, reservation: Optional[str] = None,
                   disk_size: int = 200, disk_type: Optional[str] = None, service_account_email: Optional[str] = None,
                   additional_labels: Optional[dict] = None, metadata: Optional[dict] = None,
                   compact_placement: bool = True, pre_provisioner_id: Optional[str] = None) -> dict:
    """Request body of ``nodePools.create`` for a pool of identical GPU nodes."""
    if use_spot_vm and reservation is not None:
        raise NodePoolValidationError("use_spot_vm and reservation are mutually exclusive.")
    if num_nodes < 1:
        raise NodePoolValidationError("num_nodes must be positive")
    config: dict = {"machineType": machine_type, "diskSizeGb": disk_size,
                    "oauthScopes": ["https://www.googleapis.com/auth/cloud-platform"],
                    "labels": dict(additional_labels or {}), "metadata": dict(metadata or {})}
    if accelerator:
        config["accelerators"] = [{"acceleratorCount": str(gpus_per_node), "acceleratorType": accelerator,
                                   "gpuDriverInstallationConfig": {"gpuDriverVersion": "LATEST"}}]
    if pre_provisioner_id:
        config["labels"]["pre-provisioner-id"] = pre_provisioner_id
    if use_spot_vm is not None:
        config["spot"] = bool(use_spot_vm)
    if reservation is not None:
        config["reservationAffinity"] = {"consumeReservationType": "SPECIFIC_RESERVATION",
                                         "key": "compute.googleapis.com/reservation-name", "values": [reservation]}
    if disk_type:
        config["diskType"] = disk_type
    if service_account_email:
        config["serviceAccount"] = service_account_email
    body: dict = {"nodePool": {"name": name, "initialNodeCount": num_nodes, "locations": [zone], "config": config,
                               "management": {"autoRepair": False, "autoUpgrade": False}}}
    if compact_placement and num_nodes > 1:
        body["nodePool"]["placementPolicy"] = {"type": "COMPACT"}
    return body


def get_node_pool_status(api: ContainerApi, *, project: str, zone: str, cluster: str, name: str) -> NodePoolStatus:
    pool = api.get(name=node_pool_canonical_id(project=project, zone=zone, cluster=cluster, name=name))
    if pool is None:
        return NodePoolStatus.NOT_EXIST
    try:
        return NodePoolStatus(pool.get("status", "UNKNOWN"))
    except ValueError:
        return NodePoolStatus.UNKNOWN


def _wait(predicate: Callable[[], bool], *, timeout: float, interval: float, sleep: Callable[[float], None]) -> bool:
    deadline = time.monotonic() + timeout
    while True:
        if predicate():
            return True
        if time.monotonic() >= deadline:
            return False
        sleep(interval)


def create_node_pools(api: ContainerApi, *, project: str, zone: str, cluster: str, bodies: Sequence[dict],
                      wait_timeout: float = 0, retry_interval: float = 30,
                      sleep: Callable[[float], None] = time.sleep) -> None:
    """Creates the pools that do not exist yet, then (``wait_timeout`` > 0) waits until all of them
    are RUNNING; a pool that ends in ERROR raises."""
    parent = node_pool_parent(project=project, zone=zone, cluster=cluster)
    names = [b["nodePool"]["name"] for b in bodies]
    for name, body in zip(names, bodies):
        status = get_node_pool_status(api, project=project, zone=zone, cluster=cluster, name=name)
        if status == NodePoolStatus.NOT_EXIST:
            api.create(parent=parent, body=body)
        elif status in (NodePoolStatus.STOPPING, NodePoolStatus.ERROR):
            raise NodePoolCreationError(f"node pool {name} exists in state {status.value}")
    if wait_timeout <= 0:
        return

    def ready() -> bool:
        states = [get_node_pool_status(api, project=project, zone=zone, cluster=cluster, name=n) for n in names]
        bad = [n for n, s in zip(names, states) if s in (NodePoolStatus.ERROR, NodePoolStatus.RUNNING_WITH_ERROR)]
        if bad:
            raise NodePoolCreationError(f"node pools failed to come up: {bad}")
        return all(s == NodePoolStatus.RUNNING for s in states)

    if not _wait(ready, timeout=wait_timeout, interval=retry_interval, sleep=sleep):
        raise NodePoolCreationError(f"node pools {names} not RUNNING after {wait_timeout} s")


def delete_node_pools(api: ContainerApi, *, project: str, zone: str, cluster: str, names: Sequence[str],
                      wait_timeout: float = 0, retry_interval: float = 30,
                      sleep: Callable[[float], None] = time.sleep) -> None:
    """Deletes the pools that exist (a pool that is being created is deleted once it can be), then
    optionally waits until none is left."""
    pending = list(names)

    def sweep() -> bool:
        for name in list(pending):
            status = get_node_pool_status(api, project=project, zone=zone, cluster=cluster, name=name)
            if status == NodePoolStatus.NOT_EXIST:
                pending.remove(name)
            elif status not in (NodePoolStatus.STOPPING, NodePoolStatus.PROVISIONING, NodePoolStatus.RECONCILING):
                api.delete(name=node_pool_canonical_id(project=project, zone=zone, cluster=cluster, name=name))
        return not pending

    if sweep() or wait_timeout <= 0:
        return
    if not _wait(sweep, timeout=wait_timeout, interval=retry_interval, sleep=sleep):
        raise NodePoolDeletionError(f"node pools {pending} still exist after {wait_timeout} s")


def list_node_pools_by_label_key(api: ContainerApi, *, project: str, zone: str, cluster: str, label_key: str) -> dict:
    """``{label value: [pool, ...]}`` over the cluster's pools that carry ``label_key``."""
    out: dict = {}
    for pool in api.list(parent=node_pool_parent(project=project, zone=zone, cluster=cluster)):
        value = pool.get("config", {}).get("labels", {}).get(label_key)
        if value is not None:
            out.setdefault(value, []).append(pool)
    return out
