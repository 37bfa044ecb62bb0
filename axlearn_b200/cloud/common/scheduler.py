"""Deciding which jobs run, from resource limits, project quotas and job queues.

Parity targets in the reference (axlearn/cloud/common/scheduler.py): ``ProjectJobSorter`` (:45),
``JobVerdict`` (:161), ``BaseScheduler`` / ``ScheduleResults`` (:187), ``TierScheduler`` (:427),
``JobScheduler`` (:739).

* Within a project, jobs are ordered by priority (1 first), then -- with ``use_user_usage`` -- by
  how much the submitting user already has ahead in the queue (users with less go first), then by
  creation time.
* Resources come in tiers (e.g. reserved, then pre-emptible capacity).  Project quotas are shares
  of the total, normalised to absolute amounts.  Projects take turns: the project whose usage is
  the smallest fraction of its quota goes next (ties by the creation time of its next job) and
  its next job is placed in the first tier that can hold all of its demands.  A job that fits
  nowhere gets a verdict naming the resource types that were short, and later, smaller jobs may
  still be placed (no head-of-line blocking across projects; within a project order is kept
  except that jobs too large for the whole cluster are moved to the back).
* Quotas are not hard limits: spare capacity goes to whoever asks, in the same fair order.
"""

from __future__ import annotations

import collections
import dataclasses
import datetime
from typing import Any, Mapping, Optional, Sequence

from axlearn_b200.cloud.common.job_types import JobMetadata
from axlearn_b200.cloud.common.quota import QuotaFn
from axlearn_b200.common.config import REQUIRED, Configurable, InstantiableConfig, Required, config_class, maybe_instantiate

JobQueue = list  # [(job_id, JobMetadata)]


class ProjectJobSorter(Configurable):
    @config_class
    class Config(Configurable.Config):
        use_user_usage: bool = True

    def sort(self, jobs: Mapping[str, JobMetadata]) -> JobQueue:
        by_user = collections.defaultdict(list)
        for job_id, meta in jobs.items():
            by_user[meta.user_id].append((meta.priority, meta.creation_time, job_id))
        for entries in by_user.values():
            entries.sort()
        if not self._config.use_user_usage:
            merged = sorted(e for entries in by_user.values() for e in entries)
            return [(job_id, jobs[job_id]) for _, _, job_id in merged]
        # Repeatedly take, among the users' next jobs, the one with (priority, usage so far,
        # creation time) smallest.
        usage = collections.defaultdict(int)
        cursor = {u: 0 for u in by_user}
        out = []
        while cursor:
            best = min(cursor, key=lambda u: (by_user[u][cursor[u]][0], usage[u], by_user[u][cursor[u]][1], u))
            _, _, job_id = by_user[best][cursor[best]]
            out.append((job_id, jobs[job_id]))
            usage[best] += self._aggregate_resources(jobs[job_id].resources)
            cursor[best] += 1
            if cursor[best] == len(by_user[best]):
                del cursor[best]
        return out

    def _aggregate_resources(self, resources: dict) -> int:
        return sum(resources.values())


@dataclasses.dataclass
class JobVerdict:
    over_limits: Optional[set] = None
    metadata: dict = dataclasses.field(default_factory=dict)

    def should_run(self) -> bool:
        return not self.over_limits

    def __bool__(self) -> bool:
        return self.should_run()


class BaseScheduler(Configurable):
    @dataclasses.dataclass
    class ScheduleResults:
        project_limits: dict
        project_usages: dict
        job_verdicts: dict
        unused_limits: Optional[Sequence[dict]] = None

    def schedule(self, *, resource_limits: Sequence[dict], project_quotas: dict, project_jobs: dict,
                 verbosity: int = 0) -> "BaseScheduler.ScheduleResults":
        raise NotImplementedError(type(self))


def _total(limits: Sequence[dict]) -> dict:
    out = collections.defaultdict(int)
    for tier in limits:
        for k, v in tier.items():
            out[k] += v
    return dict(out)


def _normalize_quotas(quotas: dict, totals: dict) -> dict:
    sums = collections.defaultdict(float)
    for q in quotas.values():
        for k, v in q.items():
            sums[k] += v
    return {p: {k: v / max(sums[k], 1e-8) * totals.get(k, 0) for k, v in q.items()} for p, q in quotas.items()}


class TierScheduler(BaseScheduler):
    def schedule(self, *, resource_limits, project_quotas, project_jobs, verbosity: int = 0):
        totals = _total(resource_limits)
        quotas = _normalize_quotas(project_quotas, totals)
        remaining = [dict(t) for t in resource_limits]
        usages = {p: collections.defaultdict(int) for p in project_jobs}
        queues = {}
        for project, jobs in project_jobs.items():
            fits = [(j, m) for j, m in jobs if all(v <= totals.get(k, 0) for k, v in m.resources.items())]
            rest = [(j, m) for j, m in jobs if (j, m) not in fits]
            queues[project] = collections.deque(fits + rest)
        verdicts: dict[str, JobVerdict] = {}

        def usage_ratio(project: str) -> float:
            q = quotas.get(project, {})
            ratios = []
            for k, used in usages[project].items():
                ratios.append(used / q[k] if q.get(k, 0) > 0 else (float("inf") if used > 0 else 0.0))
            nxt = queues[project][0][1]
            # Demands of the next job on resources the project has no quota for count as over-quota.
            for k, v in nxt.resources.items():
                if v > 0 and q.get(k, 0) <= 0:
                    ratios.append(float("inf"))
                elif v > 0:
                    ratios.append((usages[project][k] + v) / q[k])
            return max(ratios) if ratios else 0.0

        while any(queues.values()):
            project = min((p for p in queues if queues[p]),
                          key=lambda p: (usage_ratio(p), queues[p][0][1].creation_time, p))
            job_id, meta = queues[project].popleft()
            placed = None
            for tier, cap in enumerate(remaining):
                if all(cap.get(k, 0) >= v for k, v in meta.resources.items()):
                    placed = tier
                    break
            if placed is None:
                short = {k for k, v in meta.resources.items() if all(cap.get(k, 0) < v for cap in remaining)}
                verdicts[job_id] = JobVerdict(over_limits=short or set(meta.resources))
                continue
            for k, v in meta.resources.items():
                remaining[placed][k] -= v
                usages[project][k] += v
            verdicts[job_id] = JobVerdict(metadata={"tier": placed})
        return BaseScheduler.ScheduleResults(
            project_limits=quotas, project_usages={p: dict(u) for p, u in usages.items()},
            job_verdicts=verdicts, unused_limits=remaining)


class JobScheduler(Configurable):
    """Quota file + sorter + scheduler: ``schedule(jobs) -> ScheduleResults``; with ``dry_run``
    every job gets a should-run verdict only in the log (nothing is admitted)."""

    @config_class
    class Config(Configurable.Config):
        quota: Required[Any] = REQUIRED     # QuotaInfo, a callable returning one, or a config of such a function
        sorter: InstantiableConfig = ProjectJobSorter.default_config()
        scheduler: InstantiableConfig = TierScheduler.default_config()
        dry_run: bool = False

    def __init__(self, cfg):
        super().__init__(cfg)
        self._sorter = cfg.sorter.instantiate()
        self._scheduler = cfg.scheduler.instantiate()

    def schedule(self, jobs: Mapping[str, JobMetadata], *, dry_run: Optional[bool] = None, verbosity: int = 0):
        # The quota file is read afresh on every pass, so edits take effect without a restart.
        source = self._config.quota
        if isinstance(source, InstantiableConfig):
            info = source.instantiate()
        else:
            info = source() if callable(source) else source
        by_project = collections.defaultdict(dict)
        for job_id, meta in jobs.items():
            by_project[meta.project_id][job_id] = meta
        project_jobs = {p: self._sorter.sort(js) for p, js in by_project.items()}
        results = self._scheduler.schedule(
            resource_limits=info.total_resources, project_quotas=info.project_resources,
            project_jobs=project_jobs, verbosity=verbosity)
        if self._config.dry_run if dry_run is None else dry_run:
            results.job_verdicts = {j: JobVerdict() for j in results.job_verdicts}
        return results
