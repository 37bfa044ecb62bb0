"""Object-storage helpers over the ``gcloud storage`` CLI (reference: axlearn/cloud/gcp/storage.py:1-181,
which uses the google-cloud-storage client).  Every call goes through a runner (argument list in,
object with ``stdout`` / ``returncode`` out), so the helpers are tested without credentials and
work wherever the CLI is installed."""

from __future__ import annotations

import subprocess
from typing import Callable, Optional

Runner = Callable[..., object]


def _run(args, **kwargs):
    return subprocess.run(list(args), capture_output=True, text=True, check=False, **kwargs)


def _checked(out, what: str) -> str:
    if getattr(out, "returncode", 0) != 0:
        raise RuntimeError(f"{what} failed: {getattr(out, 'stderr', '')}".strip())
    return getattr(out, "stdout", "") or ""


def split_url(url: str) -> tuple[str, str]:
    """``gs://bucket/a/b`` -> ``("bucket", "a/b")``."""
    if not url.startswith("gs://"):
        raise ValueError(f"not a gs:// url: {url!r}")
    bucket, _, path = url[len("gs://"):].partition("/")
    if not bucket:
        raise ValueError(f"no bucket in {url!r}")
    return bucket, path


def list_blobs(url: str, *, recursive: bool = True, runner: Optional[Runner] = None) -> list[str]:
    """Object urls under ``url`` (sorted); an absent prefix lists as empty."""
    split_url(url)
    pattern = url.rstrip("/") + ("/**" if recursive else "/*")
    out = (runner or _run)(["gcloud", "storage", "ls", pattern])
    if getattr(out, "returncode", 0) != 0:
        return []       # "One or more URLs matched no objects"
    return sorted(line.strip() for line in (out.stdout or "").splitlines()
                  if line.strip() and not line.strip().endswith((":", "/")))


def blob_exists(url: str, *, runner: Optional[Runner] = None) -> bool:
    split_url(url)
    out = (runner or _run)(["gcloud", "storage", "ls", url])
    return getattr(out, "returncode", 0) == 0 and bool((out.stdout or "").strip())


def upload_blob(local_path: str, url: str, *, runner: Optional[Runner] = None) -> None:
    split_url(url)
    _checked((runner or _run)(["gcloud", "storage", "cp", local_path, url]), f"upload to {url}")


def download_blob(url: str, local_path: str, *, runner: Optional[Runner] = None) -> None:
    split_url(url)
    _checked((runner or _run)(["gcloud", "storage", "cp", url, local_path]), f"download of {url}")


def delete_blob(url: str, *, recursive: bool = False, runner: Optional[Runner] = None) -> None:
    """Deletes an object (or, with ``recursive``, everything under the prefix)."""
    split_url(url)
    cmd = ["gcloud", "storage", "rm"] + (["--recursive"] if recursive else []) + [url]
    _checked((runner or _run)(cmd), f"delete of {url}")


def sync_directory(src: str, dst: str, *, delete_unmatched: bool = False, runner: Optional[Runner] = None) -> None:
    """``gcloud storage rsync`` between a local directory and a prefix (either direction)."""
    cmd = ["gcloud", "storage", "rsync", "--recursive"] + (["--delete-unmatched-destination-objects"]
                                                           if delete_unmatched else []) + [src, dst]
    _checked((runner or _run)(cmd), f"sync {src} -> {dst}")
