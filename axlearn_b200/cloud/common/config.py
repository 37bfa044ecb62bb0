"""Per-user / per-repository settings files for the command-line tools.

Parity target: axlearn/cloud/common/config.py (``load_configs`` :30, ``update_configs`` :94, the
search of ``.axlearn/axlearn.default.config`` in the repository root and of a user file in
``./.axlearn/.axlearn.config`` or ``~/.axlearn.config``) and axlearn/cloud/gcp/config.py
(``gcp_settings`` :105: the ``[gcp]`` namespace holds one table per ``"project:env_id"`` plus
``_active``).  Files are TOML; a user file overrides the default file key by key.
"""

from __future__ import annotations

import os
import tomllib
from typing import Any, Optional, Sequence

CONFIG_DIR = ".axlearn"
DEFAULT_CONFIG_FILE = "axlearn.default.config"
CONFIG_FILE = ".axlearn.config"


def _merge(base: dict, override: dict) -> dict:
    for k, v in override.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            _merge(base[k], v)
        else:
            base[k] = v
    return base


def _repo_root_or_cwd(start: Optional[str] = None) -> str:
    path = os.path.abspath(start or os.getcwd())
    probe = path
    while True:
        if os.path.isdir(os.path.join(probe, ".git")) or os.path.isdir(os.path.join(probe, CONFIG_DIR)):
            return probe
        parent = os.path.dirname(probe)
        if parent == probe:
            return path
        probe = parent


def config_search_paths(start: Optional[str] = None) -> Sequence[str]:
    return [os.path.join(_repo_root_or_cwd(start), CONFIG_DIR, CONFIG_FILE),
            os.path.join(os.path.expanduser("~"), CONFIG_FILE)]


def load_configs(namespace: Optional[str] = None, *, required: bool = False, start: Optional[str] = None) -> tuple:
    """``(config file used, configs)``: the default file of the repository, overridden by the first
    user file found.  ``required`` raises ``SystemExit`` when no file exists."""
    configs: dict = {}
    used = None
    default = os.path.join(_repo_root_or_cwd(start), CONFIG_DIR, DEFAULT_CONFIG_FILE)
    if os.path.exists(default):
        with open(default, "rb") as f:
            _merge(configs, tomllib.load(f))
        used = default
    for path in config_search_paths(start):
        if os.path.exists(path):
            with open(path, "rb") as f:
                _merge(configs, tomllib.load(f))
            used = path
            break
    if required and used is None:
        raise SystemExit(f"A config file could not be found; create one in one of: {list(config_search_paths(start))}")
    if namespace is not None:
        configs = configs.get(namespace, {})
    return used, configs


def _toml_value(v: Any) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return str(v)
    if isinstance(v, (list, tuple)):
        return "[" + ", ".join(_toml_value(x) for x in v) + "]"
    return '"' + str(v).replace("\\", "\\\\").replace('"', '\\"') + '"'


def dump_toml(configs: dict, prefix: str = "") -> str:
    lines, tables = [], []
    for k, v in configs.items():
        key = k if k.replace("_", "").replace("-", "").isalnum() else '"' + k + '"'
        if isinstance(v, dict):
            tables.append((f"{prefix}{key}", v))
        else:
            lines.append(f"{key} = {_toml_value(v)}")
    out = "\n".join(lines)
    for name, table in tables:
        body = dump_toml(table, prefix=name + ".")
        out += ("\n\n" if out else "") + f"[{name}]\n" + body
    return out


def update_configs(namespace: str, namespace_configs: dict, *, start: Optional[str] = None) -> str:
    """Writes ``namespace_configs`` under ``[namespace]`` of the user file (created when absent)."""
    path = next((p for p in config_search_paths(start) if os.path.exists(p)), config_search_paths(start)[0])
    configs: dict = {}
    if os.path.exists(path):
        with open(path, "rb") as f:
            configs = tomllib.load(f)
    configs[namespace] = namespace_configs
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w", encoding="utf-8") as f:
        f.write("# Settings of the axlearn_b200 command-line tools.\n" + dump_toml(configs) + "\n")
    return path


def gcp_settings(key: str, *, project: Optional[str] = None, env_id: Optional[str] = None, default: Any = None,
                 required: bool = True, start: Optional[str] = None) -> Any:
    """One value of the ``[gcp."project:env_id"]`` table (the ``_active`` one when project / env_id
    are not given).  ``project`` / ``env_id`` themselves come from the arguments when set."""
    if key == "project" and project:
        return project
    if key == "env_id" and env_id:
        return env_id
    required = required and default is None
    path, configs = load_configs("gcp", required=required, start=start)
    name = f"{project}:{env_id}" if project and env_id else configs.get("_active")
    table = configs.get(name, {}) if name else {}
    if required and not table:
        raise SystemExit(f"Unknown settings for project={project} env_id={env_id}; configure the project in {path}")
    value = table.get(key, default)
    if key == "env_id" and value is None:
        value = table.get("zone")          # older files only have the zone
    if required and value is None:
        raise SystemExit(f'{path}: no value for "{key}" under [gcp."{name}"]')
    return value
