"""Job validators run by the bastion before it admits a job (reference: axlearn/cloud/common/validator.py:9-14)."""

from __future__ import annotations

import re
from typing import Optional, Sequence

from axlearn_b200.cloud.common.job_types import JobSpec
from axlearn_b200.common.config import Configurable, config_class


class ValidationError(ValueError):
    """The job must not be admitted; the message is shown to the submitter."""


class JobValidator(Configurable):
    def validate(self, job: JobSpec) -> None:
        """Raises ``ValidationError`` if ``job`` is not acceptable."""
        raise NotImplementedError(type(self))


class CompositeValidator(JobValidator):
    @config_class
    class Config(JobValidator.Config):
        validators: Sequence = ()

    def __init__(self, cfg):
        super().__init__(cfg)
        self._validators = [v.instantiate() for v in self._config.validators]

    def validate(self, job: JobSpec) -> None:
        for v in self._validators:
            v.validate(job)


class ResourceLimitValidator(JobValidator):
    """Rejects jobs whose resource request exceeds a per-job ceiling or names an unknown
    resource type, and commands that match a deny pattern."""

    @config_class
    class Config(JobValidator.Config):
        max_resources: dict = {}
        denied_command_regex: Optional[str] = None

    def validate(self, job: JobSpec) -> None:
        cfg = self._config
        for rtype, amount in (job.metadata.resources or {}).items():
            if cfg.max_resources and rtype not in cfg.max_resources:
                raise ValidationError(f"job {job.name}: unknown resource type {rtype!r}")
            if rtype in cfg.max_resources and amount > cfg.max_resources[rtype]:
                raise ValidationError(
                    f"job {job.name}: {amount} x {rtype} exceeds the per-job limit {cfg.max_resources[rtype]}")
        if cfg.denied_command_regex and re.search(cfg.denied_command_regex, job.command or ""):
            raise ValidationError(f"job {job.name}: the command matches the deny pattern")
