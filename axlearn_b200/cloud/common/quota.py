"""Project quotas and memberships read from a quota file.

Parity target in the reference: axlearn/cloud/common/quota.py (``QuotaInfo`` :20,
``get_resource_limits`` :50, ``get_user_projects`` :77).  The file is JSON (or TOML where
``tomllib`` reads it) with::

    {"total_resources": [{"b200": 64}, {"b200": 32}],        # one map per tier
     "project_resources": {"team-a": {"b200": 0.5}, ...},    # shares, normalised by the scheduler
     "project_membership": {"team-a": ["alice", "bob.*"]}}   # regexes on user ids
"""

from __future__ import annotations

import dataclasses
import json
import re
from typing import Callable, Sequence


@dataclasses.dataclass
class QuotaInfo:
    total_resources: Sequence[dict]
    project_resources: dict
    project_membership: dict

    def user_projects(self, user_id: str) -> list[str]:
        return [project for project, members in self.project_membership.items()
                if any(re.fullmatch(m, user_id) for m in members)]


QuotaFn = Callable[[], QuotaInfo]


def _load(path: str) -> dict:
    if path.endswith(".toml"):
        import tomllib

        with open(path, "rb") as f:
            d = tomllib.load(f)
        # The reference nests the tables under [toml-schema] / [total_resources] etc.; accept both.
        return d
    with open(path, encoding="utf-8") as f:
        return json.load(f)


def get_resource_limits(path: str) -> QuotaInfo:
    d = _load(path)
    total = d["total_resources"]
    if isinstance(total, dict):
        total = [total]
    return QuotaInfo(total_resources=list(total), project_resources=d.get("project_resources", {}),
                     project_membership=d.get("project_membership", {}))


def get_user_projects(path: str, user_id: str) -> list[str]:
    return get_resource_limits(path).user_projects(user_id)
