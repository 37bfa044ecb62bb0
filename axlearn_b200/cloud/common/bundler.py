"""Bundling the source tree so that a job runs the code it was submitted with.

Parity target in the reference: axlearn/cloud/common/bundler.py (``Bundler`` :60, ``BaseTarBundler``
:330, registry ``register_bundler`` / ``get_bundler_config`` :280-327).  The docker / artifact
registry / cloud-build bundlers of the reference have no counterpart: a bundle here is a
``.tar.gz`` under a (shared) directory, unpacked by the job before it starts.
"""

from __future__ import annotations

import fnmatch
import os
import tarfile
from typing import Optional, Sequence

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class

_bundlers: dict[str, type] = {}


def register_bundler(cls):
    _bundlers[cls.TYPE] = cls
    return cls


def get_bundler_config(*, bundler_type: str, spec: Sequence[str] = ()) -> "Bundler.Config":
    """``spec`` entries are ``key=value`` strings applied to the bundler's config (comma lists for
    sequence fields)."""
    if bundler_type not in _bundlers:
        raise NotImplementedError(f"unknown bundler type {bundler_type!r}; known: {sorted(_bundlers)}")
    cfg = _bundlers[bundler_type].default_config()
    for item in spec:
        key, _, value = item.partition("=")
        current = getattr(cfg, key)
        setattr(cfg, key, value.split(",") if isinstance(current, (list, tuple)) else value)
    return cfg


class Bundler(Configurable):
    TYPE = "base"

    @config_class
    class Config(Configurable.Config):
        # Glob patterns (relative paths) left out of the bundle.
        exclude: Sequence[str] = (".git", "__pycache__", "*.pyc", "_work", "*.ncu-rep")
        # Extra files or directories outside the tree to include (copied under their basename).
        external: Sequence[str] = ()

    def id(self, name: str) -> str:
        raise NotImplementedError(type(self))

    def bundle(self, name: str, *, src_dir: str = ".") -> str:
        raise NotImplementedError(type(self))

    def _included(self, rel: str) -> bool:
        parts = rel.split(os.sep)
        for pat in self._config.exclude:
            if fnmatch.fnmatch(rel, pat) or any(fnmatch.fnmatch(p, pat) for p in parts):
                return False
        return True


@register_bundler
class TarBundler(Bundler):
    TYPE = "tar"

    @config_class
    class Config(Bundler.Config):
        remote_dir: Required[str] = REQUIRED

    def id(self, name: str) -> str:
        return os.path.join(self._config.remote_dir, f"{name}.tar.gz")

    def bundle(self, name: str, *, src_dir: str = ".") -> str:
        cfg = self._config
        os.makedirs(cfg.remote_dir, exist_ok=True)
        out = self.id(name)
        tmp = out + ".tmp"
        with tarfile.open(tmp, "w:gz") as tar:
            for root, dirs, files in os.walk(src_dir):
                rel_root = os.path.relpath(root, src_dir)
                dirs[:] = [d for d in dirs if self._included(os.path.normpath(os.path.join(rel_root, d)))]
                for f in sorted(files):
                    rel = os.path.normpath(os.path.join(rel_root, f))
                    if self._included(rel):
                        tar.add(os.path.join(root, f), arcname=rel)
            for ext in cfg.external:
                tar.add(ext, arcname=os.path.basename(ext.rstrip(os.sep)))
        os.replace(tmp, out)   # readers never see a partial bundle
        return out

    @staticmethod
    def install_command(bundle_id: str, *, dest: str = ".") -> str:
        return f"mkdir -p {dest} && tar -xzf {bundle_id} -C {dest}"
