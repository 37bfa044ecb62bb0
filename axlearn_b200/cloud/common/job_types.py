"""Plain data types shared by the quota, scheduler and bastion modules.

Parity target in the reference: axlearn/cloud/common/job_types.py (``JobMetadata``, ``JobSpec``,
resource maps).  A resource map is ``{resource_type: amount}``, e.g. ``{"b200": 16}``.
"""

from __future__ import annotations

import dataclasses
import datetime
import json
from typing import Any, Optional

ResourceMap = dict
ProjectResourceMap = dict


@dataclasses.dataclass
class Topology:
    """``replicas`` copies of an accelerator topology (e.g. ``"8x8"`` GPUs x nodes of one NVLink domain)."""

    topology: str
    replicas: int


# Stands in for ``ScalingSpec.name`` when that is not set.
DEFAULT_SCALING_SPEC_NAME = "default"


@dataclasses.dataclass
class ScalingSpec:
    """Scaling bounds of one scaling group of an elastic job: it runs with any replica count in
    ``[min_replicas, max_replicas]``, each replica needing ``resources_per_replica``."""

    min_replicas: int
    max_replicas: int
    init_replicas: Optional[int] = None
    resources_per_replica: dict = dataclasses.field(default_factory=dict)
    topology_per_replica: Optional[str] = None
    name: Optional[str] = None


@dataclasses.dataclass
class JobMetadata:
    user_id: str
    project_id: str
    creation_time: datetime.datetime
    resources: dict
    priority: int = 5            # 1 = highest
    job_id: Optional[str] = None
    scaling_specs: Optional[list] = None     # list[ScalingSpec] of an elastic job

    def to_json(self) -> dict:
        d = dataclasses.asdict(self)
        d["creation_time"] = self.creation_time.isoformat()
        return d

    @classmethod
    def from_json(cls, d: dict) -> "JobMetadata":
        d = dict(d)
        d["creation_time"] = datetime.datetime.fromisoformat(d["creation_time"])
        if d.get("scaling_specs"):
            d["scaling_specs"] = [ScalingSpec(**spec) if isinstance(spec, dict) else spec for spec in d["scaling_specs"]]
        return cls(**d)


@dataclasses.dataclass
class JobSpec:
    """What the bastion needs to run a job: a shell command, an optional cleanup command, an
    environment and the scheduling metadata."""

    version: int
    name: str
    command: str
    cleanup_command: Optional[str]
    env_vars: Optional[dict]
    metadata: JobMetadata

    def to_json(self) -> dict:
        return dict(version=self.version, name=self.name, command=self.command,
                    cleanup_command=self.cleanup_command, env_vars=self.env_vars, metadata=self.metadata.to_json())

    @classmethod
    def from_json(cls, d: dict) -> "JobSpec":
        return cls(version=d["version"], name=d["name"], command=d["command"],
                   cleanup_command=d.get("cleanup_command"), env_vars=d.get("env_vars"),
                   metadata=JobMetadata.from_json(d["metadata"]))


def serialize_jobspec(spec: JobSpec, path: str) -> None:
    with open(path, "w", encoding="utf-8") as f:
        json.dump(spec.to_json(), f)


def deserialize_jobspec(path: str) -> JobSpec:
    with open(path, encoding="utf-8") as f:
        return JobSpec.from_json(json.load(f))
