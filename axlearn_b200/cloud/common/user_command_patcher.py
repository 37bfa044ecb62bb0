"""Patchers that rewrite a job's user command before it is run (reference:
axlearn/cloud/common/user_command_patcher.py)."""

from __future__ import annotations

import shlex
from typing import Any

from axlearn_b200.common.config import Configurable, config_class


class UserCommandPatcher(Configurable):
    def patch(self, command: str, **kwargs: Any) -> str:
        raise NotImplementedError(type(self))


class EnvPrefixPatcher(UserCommandPatcher):
    """Puts ``KEY=value`` assignments in front of the command: ``env_vars`` of the config, then the
    ``env_vars`` keyword of the call (e.g. what ``runtime_options.env_from_options`` returns)."""

    @config_class
    class Config(UserCommandPatcher.Config):
        env_vars: dict = {}

    def patch(self, command: str, **kwargs: Any) -> str:
        env = {**self._config.env_vars, **(kwargs.get("env_vars") or {})}
        if not env:
            return command
        return " ".join(f"{k}={shlex.quote(str(v))}" for k, v in env.items()) + " " + command
