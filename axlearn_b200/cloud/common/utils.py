"""Small helpers shared by the cloud tools (reference: axlearn/cloud/common/utils.py:68-375 and
axlearn/cloud/gcp/jobs/launch_utils.py:123-212): job names, ``key:value`` flags, list / string
canonical forms, recursive dict merge, a printable ``Table`` and the bastion's job / usage tables.
"""

from __future__ import annotations

import collections
import dataclasses
import signal
import subprocess
import uuid
from typing import Any, Callable, Optional, Sequence, Union


def generate_job_name() -> str:
    """``<user>-<5 hex digits>``: unique enough for interactive launches, short enough for the 63
    characters Kubernetes allows once suffixes are appended."""
    import getpass
    import re

    user = re.sub(r"[^a-z0-9-]", "-", getpass.getuser().lower()).strip("-") or "job"
    return f"{user}-{uuid.uuid4().hex.lower()[:5]}"


def generate_job_id() -> str:
    return str(uuid.uuid4())


def parse_kv_flags(kv_flags: Sequence[str], *, delimiter: str = ":") -> dict[str, str]:
    """``["k:v", ...] -> {k: v}``; the last occurrence of a key wins; the value may contain the delimiter."""
    out = {}
    for kv in kv_flags:
        parts = kv.split(delimiter, maxsplit=1)
        if len(parts) != 2:
            raise ValueError(f"Expected key{delimiter}value, got {kv}")
        out[parts[0]] = parts[1]
    return out


def format_table(*, headings: Sequence[str], rows: Sequence[Sequence[Any]]) -> str:
    rows = [[h.upper() for h in headings]] + [list(r) for r in rows]
    widths = [max(len(str(row[i])) for row in rows) for i in range(len(headings))]
    fmt = "".join(f"{{:<{w + 6}}}" for w in widths)
    return "\n" + "\n".join(fmt.format(*[str(v) for v in row]) for row in rows) + "\n"


def canonicalize_to_list(v: Union[str, Sequence[str], None], *, delimiter: str = ",") -> list[str]:
    if not v:
        return []                      # "".split(",") would give [""]
    if isinstance(v, str):
        v = [elem.strip() for elem in v.split(delimiter)]
    return list(v)


def canonicalize_to_string(v: Union[str, Sequence[str], None], *, delimiter: str = ",") -> str:
    if not v:
        return ""
    if not isinstance(v, str) and isinstance(v, Sequence):
        v = delimiter.join(elem.strip() for elem in v)
    return str(v)


def parse_action(argv: Sequence[str], *, options: Sequence[str], default: Optional[str] = None) -> str:
    """The first positional argument of ``argv[1:]`` if it is one of ``options``, else ``default``."""
    assert default is None or default in options
    action = next((a.strip() for a in argv[1:] if not a.strip().startswith("--")), None)
    if action not in options:
        action = default
    if action is None:
        raise ValueError(f"Invalid action: {action}. Expected one of [{', '.join(options)}].")
    return action


def merge(base: Any, overrides: dict) -> Any:
    """Recursively merges ``overrides`` into ``base`` (in place where ``base`` is a dict)."""
    if not isinstance(base, dict):
        return overrides
    for k, v in overrides.items():
        base[k] = merge(base.get(k), v) if isinstance(v, dict) else v
    return base


def to_bool(value: Any) -> bool:
    if isinstance(value, bool):
        return value
    if isinstance(value, str) and value.lower() in ("true", "false"):
        return value.lower() == "true"
    raise ValueError(f"Invalid truth value: '{value}'")


def send_signal(popen: subprocess.Popen, sig: int = signal.SIGKILL) -> None:
    """Signals a process and its descendants (children first), ignoring the ones already gone."""
    try:
        import psutil

        parent = psutil.Process(popen.pid)
        for child in parent.children(recursive=True):
            try:
                child.send_signal(sig)
            except psutil.NoSuchProcess:
                pass
    except Exception:  # pylint: disable=broad-except
        pass
    try:
        popen.send_signal(sig)
    except ProcessLookupError:
        pass


@dataclasses.dataclass(repr=False)
class Table:
    headings: list
    rows: list

    def __post_init__(self):
        for row in self.rows:
            self._check_row(row)

    def _check_row(self, row) -> None:
        if len(row) != len(self.headings):
            raise ValueError(f"Expected row to have {len(self.headings)} columns.")

    def add_row(self, row) -> None:
        self._check_row(row)
        self.rows.append(list(row))

    def add_col(self, key: str, col: Sequence[Any]) -> None:
        col = list(col)
        if self.rows and len(col) != len(self.rows):
            raise ValueError(f"Expected column to have {len(self.rows)} rows.")
        self.headings.append(key)
        if not self.rows:
            self.rows = [[v] for v in col]
        else:
            for row, v in zip(self.rows, col):
                row.append(v)

    def get_col(self, *keys: str) -> list:
        idx = [self.headings.index(k) for k in keys]
        return [[row[i] for i in idx] for row in self.rows]

    def sort(self, key: Callable[[list], Any], reverse: bool = False) -> None:
        self.rows.sort(key=key, reverse=reverse)

    def __eq__(self, other: Any) -> bool:
        return isinstance(other, Table) and other.headings == self.headings and other.rows == self.rows

    def __repr__(self) -> str:
        return format_table(headings=self.headings, rows=self.rows)


# ------------------------------------------------------------------------------------------------
# Tables over a bastion's jobs (``{name: BastionJob}``).


def jobs_table(jobs: dict) -> Table:
    return Table(
        headings=["NAME", "USER_ID", "JOB_STATE", "PROJECT_ID", "RESOURCES", "PRIORITY", "JOB_ID", "TIER"],
        rows=[[job.spec.name, job.spec.metadata.user_id, job.state.state.name, job.spec.metadata.project_id,
               str(job.spec.metadata.resources), str(job.spec.metadata.priority), job.spec.metadata.job_id,
               str(job.state.metadata.get("tier", "None"))] for job in jobs.values()])


def _usage_table(usage_info: dict) -> Table:
    table = Table(headings=["PRINCIPAL", "RESOURCE", "USAGE", "COUNT"],
                  rows=[[principal or "unknown", resource, usage[0], usage[1]]
                        for principal, per_resource in usage_info.items() for resource, usage in per_resource.items()])
    table.sort(key=lambda row: (row[1], row[2]), reverse=True)        # by resource, then usage, descending
    return table


def _usage_by(jobs: dict, principal_of: Callable[[Any], str]) -> Table:
    usage: dict = collections.defaultdict(lambda: collections.defaultdict(lambda: [0, 0]))
    for job in jobs.values():
        if job.state.state.name != "PENDING":                    # pending jobs hold nothing
            for resource, amount in job.spec.metadata.resources.items():
                entry = usage[principal_of(job)][resource]
                entry[0] += amount
                entry[1] += 1
    return _usage_table(usage)


def user_usage_table(jobs: dict) -> Table:
    return _usage_by(jobs, lambda job: job.spec.metadata.user_id)


def project_usage_table(jobs: dict) -> Table:
    return _usage_by(jobs, lambda job: job.spec.metadata.project_id)
