"""Hooks that rewrite a pod spec / a user command right before a job is submitted (reference:
axlearn/cloud/common/pod_mutator.py:12-31, user_command_patcher.py:10-22).  Deployments plug in
site policy (extra tolerations, sidecars, wrappers around the command) without touching the
job builders."""

from __future__ import annotations

import copy
from typing import Any, Optional

from axlearn_b200.cloud.common.job_types import JobSpec
from axlearn_b200.common.config import Configurable, config_class


class PodMutator(Configurable):
    def mutate(self, job_spec: Optional[JobSpec], pod: dict) -> dict:
        """Returns the pod to submit (may be ``pod`` itself, modified or not)."""
        raise NotImplementedError(type(self))


class MergePodMutator(PodMutator):
    """Deep-merges a fixed patch into every pod: dicts are merged key by key, lists are extended,
    scalars are replaced."""

    @config_class
    class Config(PodMutator.Config):
        patch: dict = {}

    def mutate(self, job_spec: Optional[JobSpec], pod: dict) -> dict:
        return _merge(copy.deepcopy(pod), self._config.patch)


def _merge(dst: Any, patch: Any) -> Any:
    if isinstance(dst, dict) and isinstance(patch, dict):
        for k, v in patch.items():
            dst[k] = _merge(dst[k], v) if k in dst else copy.deepcopy(v)
        return dst
    if isinstance(dst, list) and isinstance(patch, list):
        return dst + copy.deepcopy(patch)
    return copy.deepcopy(patch)


class UserCommandPatcher(Configurable):
    def patch(self, command: str, **kwargs) -> str:
        raise NotImplementedError(type(self))


class PrefixCommandPatcher(UserCommandPatcher):
    """``{prefix} {command}`` -- e.g. a supervising agent in front of the trainer."""

    @config_class
    class Config(UserCommandPatcher.Config):
        prefix: str = ""

    def patch(self, command: str, **kwargs) -> str:
        prefix = self._config.prefix.format(**kwargs) if kwargs else self._config.prefix
        return f"{prefix} {command}".strip()
