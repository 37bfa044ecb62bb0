"""GKE jobs: a JobSet assembled from replicated-job builders and applied through a Kubernetes API.

Parity target: axlearn/cloud/gcp/job.py (``GKEJob``: builds the JobSet custom object from a
builder, creates it through the Kubernetes custom-objects API, deletes it with foreground
propagation) and the status reading of axlearn/cloud/gcp/runners/gke.py (``GKERunnerJob.Status``
from the JobSet's conditions and per-replicated-job counters).

The Kubernetes API is an interface (``KubernetesApi``) with two implementations: ``KubectlApi``
(the ``kubectl`` binary; no client library is needed in the image) and whatever fake a test
supplies.
"""

from __future__ import annotations

import enum
import json
import subprocess
from typing import Any, Optional, Protocol

from axlearn_b200.cloud.common.job import Job
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class

JOBSET_API_VERSION = "jobset.x-k8s.io/v1alpha2"


class KubernetesApi(Protocol):
    def create_jobset(self, namespace: str, body: dict) -> Any: ...

    def get_jobset(self, namespace: str, name: str) -> Optional[dict]: ...

    def delete_jobset(self, namespace: str, name: str) -> None: ...


class KubectlApi:
    """The three calls through ``kubectl`` (JSON on stdin / stdout)."""

    def __init__(self, kubectl: str = "kubectl", context: Optional[str] = None):
        self._base = [kubectl] + (["--context", context] if context else [])

    def _run(self, args: list, *, stdin: Optional[str] = None, check: bool = True) -> subprocess.CompletedProcess:
        return subprocess.run(self._base + args, input=stdin, capture_output=True, text=True, check=check)

    def create_jobset(self, namespace: str, body: dict) -> Any:
        return self._run(["apply", "-n", namespace, "-f", "-"], stdin=json.dumps(body)).stdout

    def get_jobset(self, namespace: str, name: str) -> Optional[dict]:
        proc = self._run(["get", "jobset", name, "-n", namespace, "-o", "json"], check=False)
        if proc.returncode != 0:
            if "NotFound" in proc.stderr:
                return None
            raise RuntimeError(proc.stderr.strip())
        return json.loads(proc.stdout)

    def delete_jobset(self, namespace: str, name: str) -> None:
        self._run(["delete", "jobset", name, "-n", namespace, "--ignore-not-found", "--cascade=foreground"])


class JobSetStatus(enum.Enum):
    NOT_STARTED = "NOT_STARTED"     # no such JobSet
    PENDING = "PENDING"             # created, not all pods ready
    READY = "READY"                 # every replicated job has all its replicas ready
    SUCCEEDED = "SUCCEEDED"
    FAILED = "FAILED"
    RESCHEDULED = "RESCHEDULED"     # restarted by the JobSet failure policy at least once and not ready yet
    UNKNOWN = "UNKNOWN"


def jobset_status(jobset: Optional[dict]) -> JobSetStatus:
    """Reads a JobSet object (as returned by the API) into one status."""
    if jobset is None:
        return JobSetStatus.NOT_STARTED
    status = jobset.get("status") or {}
    for cond in status.get("conditions", []):
        if cond.get("status") == "True" and cond.get("type") == "Completed":
            return JobSetStatus.SUCCEEDED
        if cond.get("status") == "True" and cond.get("type") == "Failed":
            return JobSetStatus.FAILED
    wanted = {r["name"]: r.get("replicas", 1) for r in jobset.get("spec", {}).get("replicatedJobs", [])}
    seen = {r["name"]: r for r in status.get("replicatedJobsStatus", [])}
    if not wanted:
        return JobSetStatus.UNKNOWN
    if all(seen.get(n, {}).get("ready", 0) >= k for n, k in wanted.items()):
        return JobSetStatus.READY
    if status.get("restarts", 0) > 0:
        return JobSetStatus.RESCHEDULED
    return JobSetStatus.PENDING


class GKEJob(Job):
    """One JobSet.  ``builder`` is a replicated-job builder config (``jobset_utils``)."""

    @config_class
    class Config(Job.Config):
        builder: Required[InstantiableConfig] = REQUIRED
        namespace: str = "default"
        max_restarts: int = 0                 # whole-JobSet restarts on failure (``--max_tries``)
        queue: Optional[str] = None           # Kueue local queue
        annotations: dict = {}
        labels: dict = {}

    def __init__(self, cfg, *, api: Optional[KubernetesApi] = None, bundler: Any = None):
        super().__init__(cfg)
        self._api = api if api is not None else KubectlApi()
        self._builder = cfg.builder.clone(name=cfg.name).instantiate(bundler=bundler)

    @property
    def builder(self):
        return self._builder

    def build_jobset(self) -> dict:
        cfg = self._config
        annotations = {**self._builder.get_workload_annotations(), **cfg.annotations}
        labels = {**self._builder.get_workload_labels(), **cfg.labels}
        if cfg.queue:
            labels["kueue.x-k8s.io/queue-name"] = cfg.queue
        return dict(
            apiVersion=JOBSET_API_VERSION, kind="JobSet",
            metadata=dict(name=cfg.name, namespace=cfg.namespace, annotations=annotations, labels=labels),
            spec=dict(failurePolicy={"maxRestarts": cfg.max_restarts},
                      network={"enableDNSHostnames": True, "subdomain": cfg.name},
                      replicatedJobs=list(self._builder())))

    def _execute(self) -> Any:
        return self._api.create_jobset(self._config.namespace, self.build_jobset())

    def _delete(self) -> None:
        self._api.delete_jobset(self._config.namespace, self._config.name)

    def status(self) -> JobSetStatus:
        return jobset_status(self._api.get_jobset(self._config.namespace, self._config.name))
