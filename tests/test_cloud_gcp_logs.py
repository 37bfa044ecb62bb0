"""Job logs: Cloud Logging query, console URL, kubectl route (reference: axlearn/cloud/gcp/jobs/logs.py)."""

import datetime
import types

import pytest

from axlearn_b200.cloud.gcp import logs


class FakeLoggingClient:
    def __init__(self, entries):
        self.entries, self.calls = entries, []

    def list_entries(self, *, filter_, order_by, max_results):
        self.calls.append((filter_, order_by, max_results))
        ordered = sorted(self.entries, key=lambda e: e.timestamp, reverse=order_by == logs.DESCENDING)
        return iter(ordered[:max_results])


def _entry(minute, payload):
    return types.SimpleNamespace(timestamp=datetime.datetime(2024, 5, 1, 12, minute, 0), payload=payload)


def test_filter_and_url():
    f = logs.log_filter(name="job", worker=3, replica=1, start_time="2024-05-01", end_time="2024-05-02T00:00:00Z")
    assert f == ('resource.labels.namespace_name=default AND resource.labels.container_name=job AND '
                 'labels.k8s-pod/batch_kubernetes_io/job-completion-index=3 AND '
                 'labels.k8s-pod/jobset_sigs_k8s_io/job-index=1 AND timestamp>="2024-05-01" AND '
                 'timestamp<="2024-05-02T00:00:00Z"')
    url = logs.logs_url(name="job", start_time="2024-05-01T12:00:00Z")
    assert url.startswith("https://console.cloud.google.com/logs/query;query=resource.labels.namespace_name=default%0A")
    assert "resource.labels.container_name=job%0A" in url and url.endswith(";startTime=2024-05-01T12:00:00Z")


def test_print_logs_latest_and_earliest():
    client = FakeLoggingClient([_entry(1, "a"), _entry(2, {"message": "b"}), _entry(3, {"other": 1}), _entry(4, "d")])
    lines = []
    assert logs.print_logs(client, name="job", num_lines=3, out=lines.append) == 3
    assert client.calls[0][1:] == (logs.DESCENDING, 3)
    assert [l.split(" ", 2)[2] for l in lines[:3]] == ["b", "", "d"]          # the newest three, oldest first
    assert "startTime=2024-05-01T12:02:00Z;endTime=2024-05-01T12:04:00Z" in lines[-1]
    lines.clear()
    logs.print_logs(client, name="job", num_lines=2, earliest=True, out=lines.append)
    assert [l.split(" ", 2)[2] for l in lines[:2]] == ["a", "b"]
    lines.clear()
    assert logs.print_logs(FakeLoggingClient([]), name="job", out=lines.append) == 0 and "No logs found" in lines[0]
    with pytest.raises(ValueError):
        logs.print_logs(client, name="job", num_lines=0)


def test_kubectl_route_and_cli(capsys):
    cmd = logs.kubectl_logs_command(name="job", worker=2, replica=1, namespace="ns", num_lines=50, follow=True)
    assert cmd[:4] == ["kubectl", "logs", "-n", "ns"] and cmd[-1] == "-f" and "--tail=50" in cmd
    assert "jobset.sigs.k8s.io/jobset-name=job,jobset.sigs.k8s.io/job-index=1,batch.kubernetes.io/job-completion-index=2" in cmd
    from axlearn_b200.cli.main import main

    assert main(["gcp", "logs", "--name", "job", "--worker", "1", "--dry_run"]) == 0
    out = capsys.readouterr().out
    assert "kubectl logs -n default" in out and "job-completion-index=1" in out and "Cloud logging url:" in out
