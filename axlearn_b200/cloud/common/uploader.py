"""Background upload of a job's local output directory (reference: axlearn/cloud/common/uploader.py:14-107).

The bastion runs every job with a local log / output directory; an ``Uploader`` keeps a remote
copy fresh by calling an ``upload_fn(src_dir=, dst_dir=)`` over and over in a child process until
it is cleaned up.  The default upload function mirrors a directory tree (changed files only).
"""

from __future__ import annotations

import multiprocessing
import os
import shutil
import time
from typing import Callable, Optional

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class

UploadFn = Callable[..., None]


def mirror_directory(*, src_dir: str, dst_dir: str) -> None:
    """Copies files that are new or whose size / mtime changed; never deletes at the destination."""
    for root, _, files in os.walk(src_dir):
        rel = os.path.relpath(root, src_dir)
        out_root = os.path.normpath(os.path.join(dst_dir, rel))
        os.makedirs(out_root, exist_ok=True)
        for name in files:
            src, dst = os.path.join(root, name), os.path.join(out_root, name)
            try:
                s = os.stat(src)
                if os.path.exists(dst):
                    d = os.stat(dst)
                    if d.st_size == s.st_size and d.st_mtime >= s.st_mtime:
                        continue
                tmp = dst + ".uploading"
                shutil.copy2(src, tmp)
                os.replace(tmp, dst)
            except FileNotFoundError:
                continue          # rotated or removed between the listing and the copy


def with_interval(upload_fn: UploadFn, interval_seconds: float = 10) -> UploadFn:
    """Wraps ``upload_fn`` into a loop that runs it at most once per interval, forever (the child
    process it runs in is terminated by ``Uploader.cleanup``).  A failing round is logged and the
    loop goes on: a transient storage error must not end log uploads for good."""

    def fn(*, src_dir: str, dst_dir: str, max_rounds: Optional[int] = None):
        rounds = 0
        while max_rounds is None or rounds < max_rounds:
            start = time.time()
            try:
                upload_fn(src_dir=src_dir, dst_dir=dst_dir)
            except Exception as e:  # pylint: disable=broad-except
                print(f"upload failed: {e!r}", flush=True)
            rounds += 1
            left = interval_seconds - (time.time() - start)
            if left > 0 and (max_rounds is None or rounds < max_rounds):
                time.sleep(left)

    return fn


class Uploader(Configurable):
    @config_class
    class Config(Configurable.Config):
        src_dir: Required[str] = REQUIRED
        dst_dir: Required[str] = REQUIRED
        upload_fn: UploadFn = with_interval(mirror_directory)

    def __init__(self, cfg):
        super().__init__(cfg)
        self._upload_proc: Optional[multiprocessing.Process] = None

    def __call__(self):
        """Starts the upload process if it is not running (restarting one that died)."""
        cfg = self._config
        if self._upload_proc is not None:
            if self._upload_proc.is_alive():
                return
            self._upload_proc.join()
            self._upload_proc = None
        self._upload_proc = multiprocessing.get_context("fork").Process(
            target=cfg.upload_fn, kwargs=dict(src_dir=cfg.src_dir, dst_dir=cfg.dst_dir), daemon=True)
        self._upload_proc.start()

    def cleanup(self):
        if self._upload_proc is not None:
            self._upload_proc.terminate()      # this exact child: nothing is matched by name
            self._upload_proc.join()
            self._upload_proc = None
