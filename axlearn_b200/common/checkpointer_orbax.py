"""Checkpointer with the Orbax directory protocol (reference: axlearn/common/checkpointer_orbax.py:334-627).

The reference delegates to ``orbax.checkpoint.CheckpointManager``; here the same observable
behaviour is implemented on this framework's array storage, so that tools which walk an
Orbax-managed directory find what they expect:

* a step lives in ``{dir}/step_XXXXXXXX``; while it is being written it lives in
  ``step_XXXXXXXX.orbax-checkpoint-tmp-N`` and becomes visible through ONE atomic rename
  (``atomic_rename=True``, file systems that have it), or it is written in place and committed by
  a ``commit_success.txt`` file (``atomic_rename=False``, object stores) -- the presence of an
  ``index`` item alone never means "committed" (reference docstring :337-346);
* inside a step, one sub-directory per item of the composite: ``index/metadata`` (JSON list of the
  ``(path, value-or-spec)`` entries, what the reference saves through its JSON handler) and
  ``state/`` (the arrays, in the per-tensor chunk layout of ``TensorStoreStateStorage``), plus a
  ``_CHECKPOINT_METADATA`` JSON file with the commit time;
* retention is "the last ``keep_last_n`` steps, plus every step divisible by ``keep_period``";
* ``latest_checkpointed_step.txt`` tracks the newest committed step
  (``_CheckpointManagerWithTrackerFile``, :258-331) and ``read_latest_checkpoint_from_tracker_file``
  restores from it without listing the directory;
* a step directory that exists uncommitted is either skipped (``skip_uncommitted_checkpoint``) or
  cleared and rewritten.

Saving is asynchronous exactly as in ``Checkpointer``: device-to-host copies are enqueued, worker
threads write, and process 0 finalises (metadata, rename / commit file, tracker, retention) once
every process has flushed its chunks.
"""

from __future__ import annotations

import json
import os
import shutil
import time
from typing import Any, Callable, Optional

from axlearn_b200.common.checkpointer import (
    EXACT,
    STEP_NUM_DIGITS,
    STEP_PREFIX,
    BaseCheckpointer,
    CheckpointValidationType,
    TensorStoreStateStorage,
    parse_step_from_dir,
    write_index_file,
)
from axlearn_b200.common.config import config_class
from axlearn_b200.parallel import collectives as coll

TMP_MARKER = ".orbax-checkpoint-tmp-"
COMMIT_FILE = "commit_success.txt"
TRACKER_FILE = "latest_checkpointed_step.txt"
METADATA_FILE = "_CHECKPOINT_METADATA"


def _step_name(step: int) -> str:
    if not 0 <= step < 10**STEP_NUM_DIGITS:
        raise ValueError(f"step must be in [0, 10^{STEP_NUM_DIGITS}): {step}")
    return f"{STEP_PREFIX}_{step:0{STEP_NUM_DIGITS}d}"


def _is_committed(path: str) -> bool:
    """A step directory counts once it carries its final name AND its metadata file (atomic
    rename) or the commit file (no atomic rename)."""
    name = os.path.basename(os.path.normpath(path))
    if TMP_MARKER in name or not os.path.isdir(path):
        return False
    return os.path.exists(os.path.join(path, COMMIT_FILE)) or os.path.exists(os.path.join(path, METADATA_FILE))


class OrbaxCheckpointer(BaseCheckpointer):
    """See the module docstring."""

    @config_class
    class Config(BaseCheckpointer.Config):
        keep_last_n: int = 1
        # Steps divisible by this are kept for good (the counterpart of ``keep_every_n_steps``).
        keep_period: Optional[int] = None
        validation_type: str = EXACT
        async_timeout_secs: int = 600
        max_concurrent_save_gb: Optional[float] = None
        max_concurrent_restore_gb: Optional[float] = None
        # Accepted for config compatibility: every process of this runtime reads only the chunks
        # of its own shards, so there is no replica to single out.
        enable_single_replica_ckpt_restoring: bool = False
        replica_axis_index: int = 1
        skip_uncommitted_checkpoint: bool = True
        read_latest_checkpoint_from_tracker_file: bool = False
        # False = commit with ``commit_success.txt`` instead of a rename (object stores).
        atomic_rename: bool = True

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True
        cfg = self._config
        storage_cfg = TensorStoreStateStorage.default_config().set(
            timeout_secs=cfg.async_timeout_secs, max_concurrent_gb=cfg.max_concurrent_save_gb)
        if cfg.max_concurrent_restore_gb is not None:
            storage_cfg.max_concurrent_restore_gb = cfg.max_concurrent_restore_gb
        self._storage: TensorStoreStateStorage = storage_cfg.instantiate()
        self._save_policy: Callable[..., bool] = cfg.save_policy.instantiate()
        self._last_saved_step: Optional[int] = None

    # ---------------------------------------------------------------- listing
    @classmethod
    def checkpoint_steps(cls, base_dir: str) -> list[int]:
        return [parse_step_from_dir(p) for p in cls.checkpoint_paths(base_dir)]

    @classmethod
    def checkpoint_paths(cls, base_dir: str) -> list[str]:
        """Committed step directories, oldest first."""
        if not os.path.isdir(base_dir):
            return []
        out = []
        for name in sorted(os.listdir(base_dir)):
            path = os.path.join(base_dir, name)
            if name.startswith(f"{STEP_PREFIX}_") and _is_committed(path):
                out.append(path)
        return out

    @classmethod
    def latest_checkpoint_path(cls, base_dir: str) -> Optional[str]:
        paths = cls.checkpoint_paths(base_dir)
        return paths[-1] if paths else None

    def ckpt_dir(self, step: int, dir: Optional[str] = None) -> str:  # pylint: disable=redefined-builtin
        return os.path.join(dir or self._config.dir, _step_name(step))

    @property
    def tracker_file_path(self) -> str:
        return os.path.join(self._config.dir, TRACKER_FILE)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.stop(has_exception=exc_type is not None)
        return False

    # ---------------------------------------------------------------- save
    def save(self, *, step: int, state: Any, specs: Optional[Any] = None,
             evaler_summaries: Optional[dict] = None, force: bool = False,
             pre_save_check: Optional[Callable[[], None]] = None) -> bool:
        cfg = self._config
        if not force and not self._save_policy(step=step, evaler_summaries=evaler_summaries):
            return False
        if pre_save_check is not None:
            pre_save_check()
        final = self.ckpt_dir(step)
        if _is_committed(final):
            raise ValueError(f"checkpoint {final} already exists")
        self._storage.wait_until_finished()
        work = final + f"{TMP_MARKER}0" if cfg.atomic_rename else final
        # Every process looks at the (shared) directory before anybody changes it, so all reach
        # the same verdict without a collective on the save path.
        leftovers = [final] if os.path.isdir(final) else []
        leftovers += [os.path.join(cfg.dir, n) for n in (os.listdir(cfg.dir) if os.path.isdir(cfg.dir) else [])
                      if n.startswith(_step_name(step) + TMP_MARKER)]
        coll.barrier("orbax-ckpt-scan")
        if leftovers:
            if cfg.skip_uncommitted_checkpoint:
                # An earlier incarnation of this job left the step half-written: do not spend
                # the time deleting it, skip this save.
                return False
            if coll.process_index() == 0:
                for p in leftovers:
                    shutil.rmtree(p, ignore_errors=True)
            coll.barrier("orbax-ckpt-clear")

        def finalise(*, ckpt_dir: str, step: int, entries) -> None:
            # Runs on process 0 when every process has flushed its chunks.
            write_index_file(ckpt_dir, step=step, entries=entries)        # the storage's own reader needs it
            item_dir = os.path.join(work, "index")
            os.makedirs(item_dir, exist_ok=True)
            with open(os.path.join(item_dir, "metadata"), "w", encoding="utf-8") as f:
                json.dump([["step", int(step)]] + [[k, v] for k, v in entries], f, default=str)
            meta = {"item_handlers": {"index": "JsonCheckpointHandler", "state": "PyTreeCheckpointHandler"},
                    "init_timestamp_nsecs": self._init_ns, "commit_timestamp_nsecs": time.time_ns(), "step": step}
            if cfg.atomic_rename:
                with open(os.path.join(work, METADATA_FILE), "w", encoding="utf-8") as f:
                    json.dump(meta, f)
                os.rename(work, final)
            else:
                with open(os.path.join(work, METADATA_FILE + ".partial"), "w", encoding="utf-8") as f:
                    json.dump(meta, f)
                os.rename(os.path.join(work, METADATA_FILE + ".partial"), os.path.join(work, "checkpoint_metadata.json"))
                with open(os.path.join(final, COMMIT_FILE), "w", encoding="utf-8") as f:
                    f.write(f"Checkpoint commit was successful to {final}")
            tmp = self.tracker_file_path + ".tmp"
            with open(tmp, "w", encoding="utf-8") as f:
                f.write(_step_name(step))
            os.replace(tmp, self.tracker_file_path)
            self._run_retention(newest=step)

        self._init_ns = time.time_ns()
        self._storage.save_to_dir(step=step, state=state, ckpt_dir=os.path.join(work, "state"), specs=specs,
                                  on_commit_callback=finalise)
        self._last_saved_step = step
        return True

    def wait_until_finished(self) -> None:
        self._storage.wait_until_finished()

    # ---------------------------------------------------------------- restore
    def restore(self, *, step: Optional[int] = None, state: Any, specs: Optional[Any] = None,
                validation: Optional[CheckpointValidationType] = None, device=None) -> tuple[Optional[int], Any]:
        """Restores ``step`` (default: the newest committed step, or the tracker file's step).
        Returns ``(step, state)``, or ``(None, state)`` unchanged when nothing is there."""
        cfg = self._config
        self._storage.wait_until_finished()
        if step is None:
            path = None
            if cfg.read_latest_checkpoint_from_tracker_file and os.path.exists(self.tracker_file_path):
                with open(self.tracker_file_path, encoding="utf-8") as f:
                    candidate = os.path.join(cfg.dir, f.read().strip())
                if _is_committed(candidate):
                    path = candidate
            if path is None:
                path = self.latest_checkpoint_path(cfg.dir)
            if path is None:
                return None, state
            step = parse_step_from_dir(path)
        else:
            path = self.ckpt_dir(step)
            if not _is_committed(path):
                raise ValueError(f"checkpoint {path} does not exist or is not committed")
        restored = self._storage.restore_from_dir(
            step=step, state=state, ckpt_dir=os.path.join(path, "state"), specs=specs,
            validation=validation or cfg.validation_type, device=device)
        coll.barrier("orbax-ckpt-restore")
        return step, restored

    def stop(self, *, has_exception: bool = False) -> None:
        if not has_exception:
            self._storage.wait_until_finished()

    # ---------------------------------------------------------------- retention
    def _run_retention(self, *, newest: int) -> None:
        cfg = self._config
        steps = self.checkpoint_steps(cfg.dir)
        keep = set(steps[-max(cfg.keep_last_n, 1):]) | {newest}
        if cfg.keep_period:
            keep |= {s for s in steps if s % cfg.keep_period == 0}
        for s in steps:
            if s in keep:
                continue
            path = self.ckpt_dir(s)
            # Un-commit first, so that a crash in the middle leaves no half-deleted "committed" step.
            doomed = path + f"{TMP_MARKER}gc"
            try:
                os.rename(path, doomed)
            except OSError:
                continue
            shutil.rmtree(doomed, ignore_errors=True)
