"""Logs of a GKE job (reference: axlearn/cloud/gcp/jobs/logs.py:21-131).

Two routes to the same lines:

* Cloud Logging: ``log_filter`` builds the query for one worker of one replica of a JobSet (the
  container is named after the job), ``print_logs`` reads the newest (or earliest) ``num_lines``
  entries through an injected client (``list_entries(filter_=, order_by=, max_results=)``, what the
  Cloud Logging client offers) and prints them oldest first with a console URL for the same query;
* ``kubectl_logs_command``: the equivalent ``kubectl logs`` call for a cluster one has direct
  access to (pods of a JobSet carry the jobset name, the replicated-job index and the completion
  index as labels).
"""

from __future__ import annotations

import urllib.parse
from typing import Any, Callable, Optional, Sequence

ASCENDING = "timestamp asc"
DESCENDING = "timestamp desc"


def query_eq_filters(*, name: str, worker: int = 0, replica: int = 0, namespace: str = "default") -> dict:
    return {
        "resource.labels.namespace_name": namespace,
        "resource.labels.container_name": name,
        "labels.k8s-pod/batch_kubernetes_io/job-completion-index": worker,
        "labels.k8s-pod/jobset_sigs_k8s_io/job-index": replica,
    }


def log_filter(*, name: str, worker: int = 0, replica: int = 0, namespace: str = "default",
               start_time: Optional[str] = None, end_time: Optional[str] = None) -> str:
    """Times are ``yyyy-mm-dd`` or ``yyyy-mm-ddTH:M:SZ``; a time range makes queries for old jobs
    much faster and avoids timeouts."""
    filters = [f"{k}={v}" for k, v in query_eq_filters(name=name, worker=worker, replica=replica,
                                                        namespace=namespace).items()]
    if start_time:
        filters.append(f'timestamp>="{start_time}"')
    if end_time:
        filters.append(f'timestamp<="{end_time}"')
    return " AND ".join(filters)


def logs_url(*, name: str, worker: int = 0, replica: int = 0, namespace: str = "default",
             start_time: Optional[str] = None, end_time: Optional[str] = None) -> str:
    query = "".join(urllib.parse.urlencode([(k, f"{v}\n")])
                    for k, v in query_eq_filters(name=name, worker=worker, replica=replica, namespace=namespace).items())
    url = f"https://console.cloud.google.com/logs/query;query={query}"
    if start_time:
        url += f";startTime={start_time}"
    if end_time:
        url += f";endTime={end_time}"
    return url


def print_logs(client: Any, *, name: str, worker: int = 0, replica: int = 0, namespace: str = "default",
               num_lines: int = 1000, start_time: Optional[str] = None, end_time: Optional[str] = None,
               earliest: bool = False, out: Callable[[str], None] = print) -> int:
    """Prints up to ``num_lines`` entries, oldest first; returns how many."""
    if num_lines <= 0:
        raise ValueError("--num_lines must be greater than 0")
    entries = list(client.list_entries(
        filter_=log_filter(name=name, worker=worker, replica=replica, namespace=namespace, start_time=start_time,
                           end_time=end_time),
        order_by=ASCENDING if earliest else DESCENDING, max_results=num_lines))
    if not entries:
        out("No logs found. Consider --start_time / --end_time (yyyy-mm-dd or yyyy-mm-ddTH:M:SZ) to narrow the query.")
        return 0
    ordered = entries if earliest else list(reversed(entries))
    for entry in ordered:
        message = entry.payload
        if isinstance(message, dict):
            message = message.get("message", "")
        out(f"{entry.timestamp} {message}")
    fmt = "%Y-%m-%dT%H:%M:%SZ"
    first, last = ordered[0].timestamp, ordered[-1].timestamp
    out("\nCloud logging url: " + logs_url(
        name=name, worker=worker, replica=replica, namespace=namespace,
        start_time=first.strftime(fmt) if hasattr(first, "strftime") else str(first),
        end_time=last.strftime(fmt) if hasattr(last, "strftime") else str(last)))
    return len(entries)


def kubectl_logs_command(*, name: str, worker: int = 0, replica: int = 0, namespace: str = "default",
                         num_lines: int = 1000, follow: bool = False) -> Sequence[str]:
    selector = (f"jobset.sigs.k8s.io/jobset-name={name},jobset.sigs.k8s.io/job-index={replica},"
                f"batch.kubernetes.io/job-completion-index={worker}")
    cmd = ["kubectl", "logs", "-n", namespace, "-l", selector, "-c", name, f"--tail={num_lines}"]
    if follow:
        cmd.append("-f")
    return cmd
