"""Bundlers for Google Cloud (reference: axlearn/cloud/gcp/bundler.py:79-478): a tarball in a
storage bucket, an image in Artifact Registry built locally, an image built by Cloud Build.
Every cloud command goes through an injectable runner (argument list in, ``CompletedProcess``-like
object out), so the builders are tested without credentials."""

from __future__ import annotations

import json
import subprocess
import time
from typing import Callable, Optional

from axlearn_b200.cloud.common.bundler import BaseDockerBundler, BaseTarBundler, DockerBundler, register_bundler
from axlearn_b200.common.config import config_class


def _run(args, **kwargs):
    return subprocess.run(list(args), check=True, capture_output=True, text=True, **kwargs)


@register_bundler
class GCSTarBundler(BaseTarBundler):
    """``remote_dir`` is a ``gs://bucket/path``; copies use ``gcloud storage cp``."""

    TYPE = "gcs"

    @config_class
    class Config(BaseTarBundler.Config):
        runner: Optional[Callable] = None

    def _copy_to_remote(self, *, local_path: str, remote_path: str) -> None:
        (self._config.runner or _run)(["gcloud", "storage", "cp", local_path, remote_path])

    def _copy_to_local_command(self, *, remote_bundle_id: str, local_bundle_id: str) -> str:
        return f"gcloud storage cp {remote_bundle_id} {local_bundle_id}"


@register_bundler
class ArtifactRegistryBundler(DockerBundler):
    """Local docker build, pushed to an Artifact Registry repository (the credential helper for
    the registry host is configured first)."""

    TYPE = "artifactregistry"

    def _build_and_push(self, *args, **kwargs):
        from axlearn_b200.cloud.common import docker

        cfg = self._config
        run = cfg.runner or docker._run  # pylint: disable=protected-access
        run(["gcloud", "auth", "configure-docker", cfg.repo.split("/")[0], "--quiet"])
        return super()._build_and_push(*args, **kwargs)


def region_from_worker_pool(worker_pool: str) -> Optional[str]:
    """``projects/P/locations/REGION/workerPools/W`` -> ``REGION``."""
    parts = worker_pool.split("/")
    if len(parts) == 6 and parts[0] == "projects" and parts[2] == "locations" and parts[4] == "workerPools":
        return parts[3]
    return None


@register_bundler
class CloudBuildBundler(BaseDockerBundler):
    """Submits the build context to Cloud Build (no local docker daemon needed) and, unless
    ``is_async``, polls until the build has finished."""

    TYPE = "cloudbuild"

    @config_class
    class Config(BaseDockerBundler.Config):
        project: Optional[str] = None
        is_async: bool = False
        private_worker_pool: Optional[str] = None
        # Kaniko layer cache instead of ``--cache-from``.
        use_kaniko: bool = False
        poll_seconds: float = 10.0
        timeout_seconds: float = 3600.0
        runner: Optional[Callable] = None

    def build_config(self, *, dockerfile: str, image: str, args: dict, labels: dict) -> dict:
        """The ``cloudbuild.yaml`` content as a dict (written as JSON, which the service accepts)."""
        cfg = self._config
        import os

        name = os.path.basename(dockerfile)
        if cfg.use_kaniko:
            step_args = [f"--dockerfile={name}", f"--destination={image}", "--cache=true"]
            step_args += [f"--build-arg={k}={v}" for k, v in args.items()]
            step_args += [f"--label={k}={v}" for k, v in labels.items()]
            if cfg.target:
                step_args.append(f"--target={cfg.target}")
            steps = [{"name": "gcr.io/kaniko-project/executor:latest", "args": step_args}]
            images = []
        else:
            step_args = ["build", "-f", name, "-t", image]
            for k, v in args.items():
                step_args += ["--build-arg", f"{k}={v}"]
            for k, v in labels.items():
                step_args += ["--label", f"{k}={v}"]
            if cfg.target:
                step_args += ["--target", cfg.target]
            if cfg.platform:
                step_args += ["--platform", cfg.platform]
            for src in cfg.cache_from or ():
                step_args += ["--cache-from", src]
            steps = [{"name": "gcr.io/cloud-builders/docker", "args": step_args + ["."],
                      "env": ["DOCKER_BUILDKIT=1"]}]
            images = [image]
        out = {"steps": steps, "images": images, "timeout": f"{int(cfg.timeout_seconds)}s",
               "options": {"logging": "CLOUD_LOGGING_ONLY"}}
        if cfg.private_worker_pool:
            out["options"]["pool"] = {"name": cfg.private_worker_pool}
        return out

    def _build_and_push(self, *, dockerfile: str, image: str, args: dict, context: str, labels: dict) -> str:
        import os

        cfg = self._config
        run = cfg.runner or _run
        config_path = os.path.join(context, "cloudbuild.json")
        with open(config_path, "w", encoding="utf-8") as f:
            json.dump(self.build_config(dockerfile=dockerfile, image=image, args=args, labels=labels), f)
        cmd = ["gcloud", "builds", "submit", context, "--config", config_path, "--async", "--format", "value(id)"]
        if cfg.project:
            cmd += ["--project", cfg.project]
        region = region_from_worker_pool(cfg.private_worker_pool) if cfg.private_worker_pool else None
        if region:
            cmd += ["--region", region]
        build_id = run(cmd).stdout.strip()
        if not cfg.is_async:
            self.wait_until_finished(build_id, region=region)
        return image

    def wait_until_finished(self, build_id: str, *, region: Optional[str] = None) -> None:
        cfg = self._config
        run = cfg.runner or _run
        deadline = time.time() + cfg.timeout_seconds
        while True:
            cmd = ["gcloud", "builds", "describe", build_id, "--format", "value(status)"]
            if cfg.project:
                cmd += ["--project", cfg.project]
            if region:
                cmd += ["--region", region]
            status = run(cmd).stdout.strip()
            if status == "SUCCESS":
                return
            if status in ("FAILURE", "INTERNAL_ERROR", "TIMEOUT", "CANCELLED", "EXPIRED"):
                raise RuntimeError(f"Cloud Build {build_id} ended with status {status}")
            if time.time() > deadline:
                raise TimeoutError(f"Cloud Build {build_id} still {status} after {cfg.timeout_seconds}s")
            time.sleep(cfg.poll_seconds)
