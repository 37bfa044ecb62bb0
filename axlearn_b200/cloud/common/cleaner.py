"""Deciding which finished or unschedulable jobs can be cleaned up.

Parity target in the reference: axlearn/cloud/common/cleaner.py (``Cleaner.sweep`` returns the
names of jobs whose resources are fully released; ``UnschedulableCleaner`` sweeps jobs that could
never be scheduled with the whole cluster free).
"""

from __future__ import annotations

from typing import Mapping, Sequence

from axlearn_b200.cloud.common.job_types import JobSpec
from axlearn_b200.cloud.common.scheduler import JobScheduler
from axlearn_b200.common.config import REQUIRED, Configurable, InstantiableConfig, Required, config_class


class Cleaner(Configurable):
    def sweep(self, jobs: Mapping[str, JobSpec]) -> Sequence[str]:
        raise NotImplementedError(type(self))


class UnschedulableCleaner(Cleaner):
    @config_class
    class Config(Cleaner.Config):
        scheduler: Required[InstantiableConfig] = REQUIRED

    def __init__(self, cfg):
        super().__init__(cfg)
        self._scheduler: JobScheduler = cfg.scheduler.instantiate()

    def sweep(self, jobs):
        out = []
        for name, spec in jobs.items():
            verdict = self._scheduler.schedule({name: spec.metadata}).job_verdicts[name]
            if not verdict:
                out.append(name)
        return out
