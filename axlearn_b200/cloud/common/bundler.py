"""Bundling the source tree so that a job runs the code it was submitted with.

Parity target in the reference: axlearn/cloud/common/bundler.py (``Bundler`` :88,
``BaseDockerBundler`` :278, ``DockerBundler`` :491, ``BaseTarBundler`` :531, registry
``register_bundler`` / ``get_bundler_config`` :272, :670).  Two families: a ``.tar.gz`` of the
source tree under a (shared or remote) directory, unpacked by the job before it starts, and a
container image built from the tree and pushed to a registry.  Both copy the tree into a scratch
directory first (exclusions applied, git summary files added), so what is bundled is exactly
what a job later sees.
"""

from __future__ import annotations

import contextlib
import fnmatch
import os
import shutil
import tarfile
import tempfile
from typing import Callable, Optional, Sequence

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


class _TreeMixin:
    """Copies the (filtered) source tree plus git summary files into a scratch directory."""

    @contextlib.contextmanager
    def _local_dir_context(self, src_dir: str):
        from axlearn_b200.cloud.common.git_summary import GitSummary

        with tempfile.TemporaryDirectory(prefix="axb-bundle-") as tmp:
            root = os.path.join(tmp, "axlearn")
            os.makedirs(root)
            for cur, dirs, files in os.walk(src_dir):
                rel_root = os.path.relpath(cur, src_dir)
                dirs[:] = [d for d in dirs if self._included(os.path.normpath(os.path.join(rel_root, d)))]
                for f in files:
                    rel = os.path.normpath(os.path.join(rel_root, f))
                    if self._included(rel):
                        os.makedirs(os.path.dirname(os.path.join(root, rel)) or root, exist_ok=True)
                        shutil.copy2(os.path.join(cur, f), os.path.join(root, rel))
            for ext in self._config.external:
                dst = os.path.join(root, os.path.basename(ext.rstrip(os.sep)))
                if os.path.isdir(ext):
                    shutil.copytree(ext, dst, dirs_exist_ok=True)
                else:
                    shutil.copy2(ext, dst)
            summary = GitSummary(path=src_dir)
            if summary.is_valid():
                summary.to_disk(root)
            yield root, summary


class BaseDockerBundler(_TreeMixin, Bundler):
    """Bundles the tree into a container image; subclasses implement ``_build_and_push``."""

    TYPE = "base_docker"

    @config_class
    class Config(Bundler.Config):
        image: Required[str] = REQUIRED
        repo: Required[str] = REQUIRED
        dockerfile: Required[str] = REQUIRED
        build_args: dict = {}
        target: Optional[str] = None
        platform: Optional[str] = "linux/amd64"
        # Bundling a checkout with uncommitted changes is refused unless this is set.
        allow_dirty: bool = False
        cache_from: Optional[Sequence[str]] = None
        # Use a pre-built image: ``bundle`` only returns its id.
        skip_bundle: bool = False
        # Build targets of the same Dockerfile that are built and pushed as images of their own.
        sidecars: Sequence[str] = ()

    def __init__(self, cfg):
        super().__init__(cfg)
        cfg = self._config
        if cfg.skip_bundle:
            return
        for field in ("image", "repo", "dockerfile"):
            value = getattr(cfg, field)
            if not value or value is REQUIRED:
                raise ValueError(f"{field} cannot be empty; pass --bundler_spec={field}=...")

    def id(self, name: str) -> str:
        cfg = self._config
        return f"{cfg.repo}/{cfg.image}:{name}"

    def bundle(self, name: str, *, src_dir: str = ".") -> str:
        cfg = self._config
        if cfg.skip_bundle:
            return self.id(name)
        dockerfile = os.path.abspath(os.path.expanduser(cfg.dockerfile))
        with self._local_dir_context(src_dir) as (root, summary):
            if summary.is_valid() and summary.is_dirty() and not cfg.allow_dirty:
                raise RuntimeError("Please commit your changes or gitignore them (or set allow_dirty).")
            local_dockerfile = os.path.join(root, os.path.basename(dockerfile))
            shutil.copy2(dockerfile, local_dockerfile)
            labels = dict(summary.to_labels()) if summary.is_valid() else {}
            args = {k: (",".join(v) if isinstance(v, (list, tuple)) else str(v)) for k, v in cfg.build_args.items()}
            return self._build_and_push(dockerfile=local_dockerfile, image=self.id(name), args=args, context=root,
                                        labels=labels)

    @staticmethod
    def install_command(bundle_id: str) -> str:
        return f"docker pull {bundle_id}"

    def _build_and_push(self, *, dockerfile: str, image: str, args: dict, context: str, labels: dict) -> str:
        raise NotImplementedError(type(self))


@register_bundler
class DockerBundler(BaseDockerBundler):
    """Builds with the local docker daemon and pushes to ``repo``."""

    TYPE = "docker"

    @config_class
    class Config(BaseDockerBundler.Config):
        # Command runner (argument list, **kwargs); tests pass a recorder.
        runner: Optional[Callable] = None

    def _build_and_push(self, *, dockerfile: str, image: str, args: dict, context: str, labels: dict) -> str:
        from axlearn_b200.cloud.common import docker

        cfg = self._config
        run = cfg.runner or docker._run  # pylint: disable=protected-access
        tag = image.rsplit(":", maxsplit=1)[1]
        for sidecar in cfg.sidecars:
            side_image = f"{cfg.repo}/{sidecar}:{tag}"
            docker.push(docker.build(dockerfile=dockerfile, image=side_image, args=args, context=context,
                                     target=sidecar, labels=labels, platform=cfg.platform,
                                     cache_from=cfg.cache_from, runner=run), runner=run)
        return docker.push(docker.build(dockerfile=dockerfile, image=image, args=args, context=context,
                                        target=cfg.target, labels=labels, platform=cfg.platform,
                                        cache_from=cfg.cache_from, runner=run), runner=run)


class BaseTarBundler(_TreeMixin, Bundler):
    """Packs the scratch copy of the tree into ``{remote_dir}/{name}/axlearn.tar.gz`` through a
    ``_copy_to_remote`` that subclasses provide (a mounted path, an object store, ...)."""

    TYPE = "base_tar"

    @config_class
    class Config(Bundler.Config):
        remote_dir: Required[str] = REQUIRED

    def id(self, name: str) -> str:
        return f"{self._config.remote_dir.rstrip('/')}/{name}/axlearn.tar.gz"

    def bundle(self, name: str, *, src_dir: str = ".") -> str:
        with self._local_dir_context(src_dir) as (root, _):
            tar_path = os.path.join(os.path.dirname(root), "axlearn.tar.gz")
            with tarfile.open(tar_path, "w:gz") as tar:
                tar.add(root, arcname=".")
            self._copy_to_remote(local_path=tar_path, remote_path=self.id(name))
        return self.id(name)

    def _copy_to_remote(self, *, local_path: str, remote_path: str) -> None:
        raise NotImplementedError(type(self))

    def _copy_to_local_command(self, *, remote_bundle_id: str, local_bundle_id: str) -> str:
        raise NotImplementedError(type(self))

    def install_command(self, bundle_id: str, *, dest: str = ".") -> str:
        local = os.path.join(dest, "axlearn.tar.gz")
        copy = self._copy_to_local_command(remote_bundle_id=bundle_id, local_bundle_id=local)
        return f"mkdir -p {dest} && {copy} && tar -xzf {local} -C {dest}"
