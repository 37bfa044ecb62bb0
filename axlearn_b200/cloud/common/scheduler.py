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
import logging
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

    def schedule(self, jobs: Mapping[str, JobMetadata], *, dry_run: Optional[bool] = None, verbosity: int = 0,
                 desired_replicas: Optional[Mapping[str, Mapping[str, int]]] = None):
        """``desired_replicas``: ``{job: {scaling group: replicas}}`` for elastic jobs (what a
        ``ReplicaManager`` reports); without an entry an elastic job asks for its ``min_replicas``.

        An elastic job is scheduled as its base job (``metadata.resources``: the minimum it runs
        with) plus one expansion slot per replica beyond ``min_replicas``; the slots inherit the
        job's priority and age and compete with every other job.  Admitted slots are folded back
        into the parent's verdict as ``metadata["granted_replicas"]`` (always present for an
        admitted elastic job, so that a scale-down is observed too); a slot whose parent was not
        admitted is dropped."""
        # The quota file is read afresh on every pass, so edits take effect without a restart.
        source = self._config.quota
        if isinstance(source, InstantiableConfig):
            info = source.instantiate()
        else:
            info = source() if callable(source) else source
        expanded, slot_info = _expand_elastic_jobs(jobs, desired_replicas or {})
        by_project = collections.defaultdict(dict)
        for job_id, meta in expanded.items():
            by_project[meta.project_id][job_id] = meta
        project_jobs = {p: self._sorter.sort(js) for p, js in by_project.items()}
        results = self._scheduler.schedule(
            resource_limits=info.total_resources, project_quotas=info.project_resources,
            project_jobs=project_jobs, verbosity=verbosity)
        results = _collapse_expansion_verdicts(results, slot_info, jobs)
        if self._config.dry_run if dry_run is None else dry_run:
            results.job_verdicts = {j: JobVerdict() for j in results.job_verdicts}
        return results


GRANTED_REPLICAS_KEY = "granted_replicas"


def expansion_slot_name(job_name: str, spec_name: str, index: int) -> str:
    return f"{job_name}--exp-{spec_name}-{index}"


def _expand_elastic_jobs(jobs: Mapping[str, JobMetadata], desired: Mapping[str, Mapping[str, int]]):
    """``(jobs plus expansion slots, {slot: (parent job, scaling group)})``.  Stateless: every pass
    builds all slots from ``min_replicas`` up to the target afresh."""
    from axlearn_b200.cloud.common.job_types import DEFAULT_SCALING_SPEC_NAME

    expanded, slot_info = dict(jobs), {}
    for job_name, meta in jobs.items():
        for spec in getattr(meta, "scaling_specs", None) or []:
            spec_name = spec.name or DEFAULT_SCALING_SPEC_NAME
            target = min(int(desired.get(job_name, {}).get(spec_name, spec.min_replicas)), spec.max_replicas)
            for i in range(spec.min_replicas, target):
                slot = expansion_slot_name(job_name, spec_name, i)
                expanded[slot] = dataclasses.replace(meta, resources=dict(spec.resources_per_replica), scaling_specs=None)
                slot_info[slot] = (job_name, spec_name)
    return expanded, slot_info


def _collapse_expansion_verdicts(results, slot_info: Mapping[str, tuple], jobs: Mapping[str, JobMetadata]):
    from axlearn_b200.cloud.common.job_types import DEFAULT_SCALING_SPEC_NAME

    for job_name, meta in jobs.items():
        verdict = results.job_verdicts.get(job_name)
        if getattr(meta, "scaling_specs", None) and verdict:
            verdict.metadata[GRANTED_REPLICAS_KEY] = {(spec.name or DEFAULT_SCALING_SPEC_NAME): spec.min_replicas
                                                      for spec in meta.scaling_specs}
    collapsed = {}
    for name, verdict in results.job_verdicts.items():
        if name not in slot_info:
            collapsed[name] = verdict
            continue
        parent, spec_name = slot_info[name]
        parent_verdict = results.job_verdicts.get(parent)
        if not parent_verdict:
            if verdict:
                logging.warning("Expansion slot %s admitted but its parent %s is not; dropping the slot.", name, parent)
            continue
        if verdict:
            granted = parent_verdict.metadata.setdefault(GRANTED_REPLICAS_KEY, {})
            granted[spec_name] = granted.get(spec_name, 0) + 1
    results.job_verdicts = collapsed
    return results
