"""Launches a JobSet and monitors it to the end (reference: axlearn/cloud/gcp/runners/gke.py:401-889).

The runner is what a bastion starts for every scheduled job.  It polls the JobSet and acts on what
it sees:

* NOT_STARTED: wait for the image build, delete node pools which an earlier incarnation made for
  another scheduling tier, pre-provision pools, create the JobSet;
* RESCHEDULED (the bastion moved the job to another tier than the one its resources were made for):
  delete the JobSet and the mismatched node pools; the next poll starts it again;
* UPDATING (the bastion holds a newer version of the job than the one deployed): delete the JobSet;
* SUCCEEDED / COMPLETED / FAILED: publish the lifecycle event and return;
* READY / PENDING / SUSPENDED: publish once per change, keep polling.

The Kubernetes and GKE container APIs are injected (``KubernetesApi`` / ``ContainerApi``), so the
loop is tested against in-memory fakes.  The TPU-only parts of the reference (slice-selection
patching, Pathways, Flink) have no counterpart on a GPU cluster.
"""

from __future__ import annotations

import enum
import logging
import os
import time
from typing import Any, Callable, Optional

from axlearn_b200.cloud.common.event_queue import BaseQueueClient, JobLifecycleEvent
from axlearn_b200.cloud.common.job import Job
from axlearn_b200.cloud.gcp import node_pool
from axlearn_b200.cloud.gcp.job import GKEJob, KubernetesApi
from axlearn_b200.cloud.gcp.runners import utils as runner_utils
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class

BASTION_JOB_VERSION_ENV_VAR = "BASTION_JOB_VERSION"
BASTION_JOB_VERSION_LABEL = "bastion-job-version"
BASTION_TIER_ENV_VAR = "BASTION_TIER"
PRE_PROVISIONER_LABEL = "pre-provisioner-id"
AUTO_PROVISIONER_LABEL = "provisioner-nodepool-id"


class JobLifecycleState(str, enum.Enum):
    STARTING = "STARTING"
    RUNNING = "RUNNING"
    SUCCEEDED = "SUCCEEDED"
    FAILED = "FAILED"


def _pod_specs(jobset_spec: dict):
    for job in jobset_spec.get("replicatedJobs", []):
        yield job, job["template"]["spec"]["template"]


def infer_reservation(jobset_spec: dict) -> Optional[str]:
    try:
        for _, pod in _pod_specs(jobset_spec):
            name = pod["spec"].get("nodeSelector", {}).get("cloud.google.com/reservation-name")
            if name is not None:
                return name
    except (TypeError, KeyError):
        logging.warning("Failed to infer reservation.")
    return None


def infer_processor_type(jobset_spec: dict) -> Optional[str]:
    try:
        for _, pod in _pod_specs(jobset_spec):
            selector = pod["spec"].get("nodeSelector", {})
            if "cloud.google.com/gke-accelerator" in selector:
                return "gpu"
            if "cloud.google.com/gke-tpu-accelerator" in selector:
                return "tpu"
            for container in pod["spec"].get("containers", []):
                limits = container.get("resources", {}).get("limits", {})
                if "nvidia.com/gpu" in limits:
                    return "gpu"
                if "google.com/tpu" in limits:
                    return "tpu"
    except (TypeError, KeyError):
        logging.warning("Failed to infer processor type.")
    return None


def infer_job_version(jobset_spec: dict) -> Optional[int]:
    try:
        for _, pod in _pod_specs(jobset_spec):
            version = pod.get("metadata", {}).get("labels", {}).get(BASTION_JOB_VERSION_LABEL)
            if version is not None:
                return int(version)
    except (TypeError, KeyError, ValueError):
        logging.warning("Failed to infer job version.")
    return None


def infer_job_count(jobset_spec: dict) -> int:
    return sum(int(job.get("replicas", 1)) for job in jobset_spec.get("replicatedJobs", []))


def mismatched_node_pools(pools: list, *, tier: Any) -> list:
    """Pools whose capacity source does not fit the tier: tier 0 wants a reservation, every other
    tier wants spot nodes."""
    out = []
    for pool in pools:
        config = pool.get("config", {})
        affinity = config.get("reservationAffinity", {})
        has_reservation = (affinity.get("key") == "compute.googleapis.com/reservation-name"
                           and len(affinity.get("values", [])) > 0)
        has_spot = any(t.get("key") == "cloud.google.com/gke-spot" and t.get("value") == "true"
                       and t.get("effect") == "NO_SCHEDULE" for t in config.get("taints", []))
        if (str(tier) == "0" and not has_reservation) or (str(tier) != "0" and not has_spot):
            out.append(pool)
    return out


class GKERunnerJob(Job):
    class Status(enum.Enum):
        UNKNOWN = "UNKNOWN"
        NOT_STARTED = "NOT_STARTED"                 # the JobSet does not exist
        PENDING = "PENDING"                         # exists, not every job is ready
        COMPLETED = "COMPLETED"
        FAILED = "FAILED"
        SUSPENDED = "SUSPENDED"
        STARTUPPOLICYCOMPLETED = "STARTUPPOLICYCOMPLETED"
        READY = "READY"                             # every job is ready
        SUCCEEDED = "SUCCEEDED"
        UPDATING = "UPDATING"                       # will be relaunched with a newer spec
        RESCHEDULED = "RESCHEDULED"                 # was moved to another tier

    @config_class
    class Config(Job.Config):
        inner: Required[InstantiableConfig] = REQUIRED       # GKEJob.Config
        output_dir: Optional[str] = None
        project: Optional[str] = None
        zone: Optional[str] = None
        cluster: Optional[str] = None
        status_interval_seconds: float = 30
        pre_provisioner: Optional[InstantiableConfig] = None
        event_publisher: Optional[InstantiableConfig] = None
        # Stop after this many polls (None: until the job ends); for dry runs and tests.
        max_polls: Optional[int] = None

    def __init__(self, cfg, *, api: KubernetesApi, bundler: Any = None, container_api: Optional[node_pool.ContainerApi] = None,
                 event_publisher: Optional[BaseQueueClient] = None, sleep: Callable[[float], None] = time.sleep,
                 environ: Optional[dict] = None, summary_uploader: Optional[Callable[[], None]] = None):
        super().__init__(cfg)
        cfg = self._config
        self._api, self._bundler, self._container_api, self._sleep = api, bundler, container_api, sleep
        self._environ = os.environ if environ is None else environ
        self._inner: GKEJob = cfg.inner.clone(name=cfg.name).instantiate(api=api, bundler=bundler)
        self._pre_provisioner = None
        if cfg.pre_provisioner is not None:
            self._pre_provisioner = cfg.pre_provisioner.clone(name=cfg.name).instantiate(api=container_api, sleep=sleep)
        self._event_publisher = event_publisher if event_publisher is not None else (
            cfg.event_publisher.instantiate() if cfg.event_publisher is not None else None)
        self._summary_uploader = summary_uploader
        self.last_status: Optional[GKERunnerJob.Status] = None
        self.timings: dict[str, float] = {}

    @property
    def inner(self) -> GKEJob:
        return self._inner

    @property
    def is_running(self) -> bool:
        return self.last_status == GKERunnerJob.Status.READY

    # ------------------------------------------------------------------ status
    def _tier(self) -> Any:
        """The scheduling tier the bastion assigned, or None when no bastion started this runner (a
        job launched by hand is never moved between tiers, so nothing is recreated for it)."""
        return self._environ.get(BASTION_TIER_ENV_VAR)

    def _should_recreate(self, reservation, processor, *, is_pending: bool = False) -> bool:
        tier = self._tier()
        return tier is not None and runner_utils.should_recreate_job(tier, reservation, processor_type=processor,
                                                                     is_pending=is_pending)

    def _get_status(self) -> "GKERunnerJob.Status":
        cfg = self._config
        Status = GKERunnerJob.Status
        resp = self._api.get_jobset(self._inner.config.namespace, cfg.name)
        if resp is None:
            return Status.NOT_STARTED
        try:
            spec = resp["spec"]
            reservation, processor = infer_reservation(spec), infer_processor_type(spec)
            if self._should_recreate(reservation, processor):
                return Status.RESCHEDULED
            expected = self._environ.get(BASTION_JOB_VERSION_ENV_VAR)
            current = infer_job_version(spec)
            if expected is not None and (current is None or int(expected) > current):
                logging.info("Current job version is %s; expected job version is %s", current, expected)
                return Status.UPDATING
            status = resp.get("status") or {}
            # Conditions may be missing until the JobSet ends; once there they are authoritative.
            for condition in status.get("conditions", []):
                if str(condition.get("status", "")).lower() == "true":
                    logging.info("Job reached status %s with reason %s", condition["type"], condition.get("reason"))
                    return Status[condition["type"].upper()]
            counts = {k: 0 for k in ("failed", "ready", "succeeded")}
            for job in status["replicatedJobsStatus"]:
                for k in counts:
                    counts[k] += job.get(k, 0)
            total = infer_job_count(spec)
            if total and sum(counts.values()) == total and not counts["failed"]:
                for k in ("ready", "succeeded"):
                    if counts[k] == total:
                        return Status[k.upper()]
                if counts["ready"]:
                    return Status.READY
                raise RuntimeError(f"Unexpected replicatedJobsStatus: {counts}")
            if counts["failed"]:
                logging.info("One or more child jobs failed, waiting for jobset to retry.")
            if self._should_recreate(reservation, processor, is_pending=True):
                return Status.RESCHEDULED
            return Status.PENDING
        except KeyError as e:
            logging.warning("Got KeyError: %s, attempting to ignore.", e)
        return Status.UNKNOWN

    # ------------------------------------------------------------------ actions
    def _delete(self) -> None:
        self._inner._delete()  # pylint: disable=protected-access
        if self._pre_provisioner is not None:
            self._pre_provisioner.delete_for(self._inner)

    def _delete_mismatched_pools(self, label_key: str) -> list:
        cfg = self._config
        if self._container_api is None or not (cfg.project and cfg.zone and cfg.cluster):
            return []
        pools = node_pool.list_node_pools_by_label_key(
            self._container_api, project=cfg.project, zone=cfg.zone, cluster=cfg.cluster, label_key=label_key).get(cfg.name, [])
        if not pools:
            logging.info("Could not infer node pool, skipping delete.")
            return []
        tier = self._tier()
        names = [p["name"] for p in mismatched_node_pools(pools, tier=0 if tier is None else tier)]
        if names:
            start = time.perf_counter()
            node_pool.delete_node_pools(self._container_api, project=cfg.project, zone=cfg.zone, cluster=cfg.cluster,
                                        names=names, retry_interval=cfg.retry_interval,
                                        wait_timeout=30 * 60 * len(names), sleep=self._sleep)
            logging.info("Node pools %s deletion took %s seconds", names, time.perf_counter() - start)
        return names

    def _reschedule(self) -> list:
        """Deletes the JobSet and the pools made for the wrong tier, so that the provisioner makes
        them again with the right capacity source."""
        logging.info("Deleting jobset %s", self._config.name)
        self._inner._delete()  # pylint: disable=protected-access
        return self._delete_mismatched_pools(PRE_PROVISIONER_LABEL if self._pre_provisioner is not None
                                             else AUTO_PROVISIONER_LABEL)

    def _get_build_name(self) -> str:
        image_id = getattr(getattr(self._inner.builder, "config", None), "image_id", None)
        return image_id or self._config.name

    def _on_build_finished(self) -> None:
        """Hook: after the image build completed."""

    def _on_job_submitted(self) -> None:
        """Hook: after the JobSet was created."""

    def _start(self) -> bool:
        cfg = self._config
        try:
            t0 = time.perf_counter()
            if self._bundler is not None and hasattr(self._bundler, "wait_until_finished"):
                self._bundler.wait_until_finished(self._get_build_name())
            self.timings["wait_for_build"] = time.perf_counter() - t0
            self._maybe_publish(cfg.name, msg="Cloud build finished", state=JobLifecycleState.STARTING)
            self._on_build_finished()
        except RuntimeError as e:
            logging.error("Bundling failed: %s. Aborting the job.", e)
            return False
        if self._pre_provisioner is not None:
            self._delete_mismatched_pools(PRE_PROVISIONER_LABEL)
            self._pre_provisioner.create_for(self._inner)
        self._inner.execute()
        self._on_job_submitted()
        self._maybe_publish(cfg.name, msg="Provisioning resources", state=JobLifecycleState.STARTING)
        return True

    # ------------------------------------------------------------------ loop
    def _execute(self) -> Optional["GKERunnerJob.Status"]:
        cfg = self._config
        Status = GKERunnerJob.Status
        start = time.perf_counter()
        last_job_status = suspended_since = provisioning_start = None
        polls = 0
        while cfg.max_polls is None or polls < cfg.max_polls:
            polls += 1
            status = self.last_status = self._get_status()
            if status == Status.FAILED:
                self._maybe_publish(cfg.name, msg="Job failed with error", state=JobLifecycleState.FAILED)
                logging.info("Task %s exited with status: %s.", cfg.name, status)
                return status
            if status in (Status.SUCCEEDED, Status.COMPLETED):
                self._maybe_publish(cfg.name, msg="Job succeeds", state=JobLifecycleState.SUCCEEDED)
                logging.info("Task %s exited with status: %s.", cfg.name, status)
                return status
            if status == Status.RESCHEDULED:
                logging.info("RESCHEDULED detected, performing full reschedule.")
                self._reschedule()
            elif status == Status.UPDATING:
                logging.info("Newer job version is available. Relaunching the jobset...")
                self._inner._delete()  # pylint: disable=protected-access
            elif status == Status.NOT_STARTED:
                logging.info("Task has not started. Starting it now...")
                provisioning_start = time.perf_counter()
                if not self._start():
                    return None
            elif status == Status.SUSPENDED:
                if suspended_since is None:
                    suspended_since = time.perf_counter()
                    logging.info("Job %s entered SUSPENDED state", cfg.name)
            else:
                if suspended_since is not None:
                    self.timings["suspended"] = self.timings.get("suspended", 0.0) + time.perf_counter() - suspended_since
                    suspended_since = None
                if self._summary_uploader is not None:
                    self._summary_uploader()
                logging.info("Task %s has status: %s", cfg.name, status)
                if status == Status.READY and status != last_job_status:
                    self.timings["time_to_running"] = time.perf_counter() - start
                    if provisioning_start is not None:
                        self.timings["provisioning"] = time.perf_counter() - provisioning_start
                    self._maybe_publish(cfg.name, msg="Job is running", state=JobLifecycleState.RUNNING)
                    last_job_status = status
                elif status == Status.PENDING and status != last_job_status:
                    self._maybe_publish(cfg.name, msg="Job is starting", state=JobLifecycleState.STARTING)
                    last_job_status = status
            self._sleep(cfg.status_interval_seconds)
        return self.last_status

    def _maybe_publish(self, job_name: str, *, msg: str, state: JobLifecycleState) -> None:
        if self._event_publisher is None:
            return
        self._event_publisher.publish(JobLifecycleEvent(job_name=job_name, state=state.value, details=msg))
