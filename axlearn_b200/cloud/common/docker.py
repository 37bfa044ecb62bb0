"""Composing and running ``docker build`` / ``docker push`` (reference: axlearn/cloud/common/docker.py:17-95).

The commands are built as argument lists and handed to a runner (``subprocess.run`` by default),
so bundlers can be tested without a docker daemon by passing a recording runner.
"""

from __future__ import annotations

import subprocess
from typing import Callable, Optional, Sequence

Runner = Callable[..., object]


def _run(args: Sequence[str], **kwargs):
    """Runs a command; output goes to the caller's terminal (a build can be long and its progress
    matters), failures raise ``CalledProcessError``."""
    return subprocess.run(list(args), check=True, **kwargs)


def build_command(*, dockerfile: str, image: str, context: str, args: Optional[dict[str, str]] = None,
                  target: Optional[str] = None, labels: Optional[dict[str, str]] = None,
                  platform: Optional[str] = None, cache_from: Optional[Sequence[str]] = None) -> list[str]:
    cmd = ["docker", "build", "-t", image, "-f", dockerfile]
    for k, v in (args or {}).items():
        cmd += ["--build-arg", f"{k}={v}"]
    for k, v in (labels or {}).items():
        cmd += ["--label", f"{k}={v}"]
    if target:
        cmd += ["--target", target]
    if platform:
        cmd += ["--platform", platform]
    for src in cache_from or ():
        cmd += ["--cache-from", src]
    return cmd + [context]


def build(*, dockerfile: str, image: str, context: str, args: Optional[dict[str, str]] = None,
          target: Optional[str] = None, labels: Optional[dict[str, str]] = None,
          platform: Optional[str] = None, cache_from: Optional[Sequence[str]] = None,
          runner: Runner = _run) -> str:
    """Builds ``image`` from ``dockerfile`` in ``context`` with BuildKit enabled; returns the tag."""
    import os

    cmd = build_command(dockerfile=dockerfile, image=image, context=context, args=args, target=target,
                        labels=labels, platform=platform, cache_from=cache_from)
    runner(cmd, env={**os.environ, "DOCKER_BUILDKIT": "1", "BUILDKIT_PROGRESS": "plain"})
    return image


def push(image: str, *, runner: Runner = _run) -> str:
    runner(["docker", "push", image])
    return image


def registry_from_repo(repo: str) -> str:
    """``us-docker.pkg.dev/project/repo`` -> ``https://us-docker.pkg.dev`` (what ``docker login`` /
    credential helpers are configured for)."""
    return f"https://{repo.split('/')[0]}"
