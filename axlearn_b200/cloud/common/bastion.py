"""Bastion: a long-running orchestrator that admits, runs, pre-empts and cleans up jobs.

Parity target in the reference: axlearn/cloud/common/bastion.py (job states :200-260, the
directory protocol :1-79, ``Bastion.execute`` / ``_update_job`` / ``_gc_jobs`` :900-1700,
``BastionDirectory.submit_job`` / ``cancel_job`` / ``list_jobs`` :1720-1831).  The reference keeps
its state in a cloud bucket and runs on one VM; here the state lives in a directory (local disk or
a shared file system of the B200 cluster) with the same layout:

    <root>/jobs/active/<name>        serialised JobSpec of every job that is not finished
    <root>/jobs/complete/<name>      ... of finished jobs
    <root>/jobs/states/<name>        {"state": ..., "metadata": {...}} written by the bastion
    <root>/jobs/user_states/<name>   {"state": "CANCELLING"} written by users
    <root>/logs/<name>               stdout + stderr of the job's command
    <root>/logs/<name>.cleanup       ... of its cleanup command

State machine: PENDING -(scheduler says run)-> ACTIVE -(command exits)-> CLEANING -(cleanup
exits)-> COMPLETED; ACTIVE -(scheduler says stop: pre-emption)-> PENDING (the command is
terminated; it is expected to resume from its checkpoints when started again); any state
-(user cancels)-> CANCELLING -> CLEANING.  One ``execute_once`` pass: sync specs and user states
from disk, collect finished commands, schedule, start / stop commands, write states.
"""

from __future__ import annotations

import dataclasses
import enum
import json
import logging
import os
import shlex
import signal
import subprocess
import time
from typing import Any, Optional

from axlearn_b200.cloud.common.job_types import JobSpec, deserialize_jobspec, serialize_jobspec
from axlearn_b200.cloud.common.scheduler import JobScheduler
from axlearn_b200.common.config import REQUIRED, Configurable, InstantiableConfig, Required, config_class


class JobState(str, enum.Enum):
    PENDING = "PENDING"
    ACTIVE = "ACTIVE"
    CANCELLING = "CANCELLING"
    CLEANING = "CLEANING"
    COMPLETED = "COMPLETED"


@dataclasses.dataclass
class JobStatus:
    state: JobState
    metadata: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class _Running:
    process: subprocess.Popen
    log: Any


@dataclasses.dataclass
class BastionJob:
    spec: JobSpec
    state: JobStatus
    command_proc: Optional[_Running] = None
    cleanup_proc: Optional[_Running] = None


def is_valid_job_name(name: str) -> bool:
    return bool(name) and "/" not in name and not name.startswith(".") and not name.endswith(".")


class BastionDirectory(Configurable):
    """The user-side view of a bastion's directory: submit, cancel, list."""

    @config_class
    class Config(Configurable.Config):
        root_dir: Required[str] = REQUIRED

    def __init__(self, cfg):
        super().__init__(cfg)
        for d in (self.active_job_dir, self.complete_job_dir, self.job_states_dir, self.user_states_dir, self.logs_dir):
            os.makedirs(d, exist_ok=True)

    root_dir = property(lambda self: self._config.root_dir)
    active_job_dir = property(lambda self: os.path.join(self.root_dir, "jobs", "active"))
    complete_job_dir = property(lambda self: os.path.join(self.root_dir, "jobs", "complete"))
    job_states_dir = property(lambda self: os.path.join(self.root_dir, "jobs", "states"))
    user_states_dir = property(lambda self: os.path.join(self.root_dir, "jobs", "user_states"))
    logs_dir = property(lambda self: os.path.join(self.root_dir, "logs"))

    def submit_job(self, job_name: str, *, job_spec: JobSpec) -> None:
        if not is_valid_job_name(job_name):
            raise ValueError(f"invalid job name {job_name!r}")
        dst = os.path.join(self.active_job_dir, job_name)
        if os.path.exists(dst):
            logging.info("job %s exists already; not overwriting it", job_name)
            return
        tmp = dst + ".tmp"
        serialize_jobspec(job_spec, tmp)
        os.replace(tmp, dst)

    def cancel_job(self, job_name: str) -> None:
        if not os.path.exists(os.path.join(self.active_job_dir, job_name)):
            raise ValueError(f"job {job_name!r} is not active")
        with open(os.path.join(self.user_states_dir, job_name), "w", encoding="utf-8") as f:
            json.dump({"state": JobState.CANCELLING.value}, f)

    def get_job_state(self, job_name: str) -> Optional[JobStatus]:
        path = os.path.join(self.job_states_dir, job_name)
        if not os.path.exists(path):
            return None
        with open(path, encoding="utf-8") as f:
            d = json.load(f)
        return JobStatus(JobState(d["state"]), d.get("metadata", {}))

    def list_jobs(self) -> dict[str, BastionJob]:
        out = {}
        for name in sorted(os.listdir(self.active_job_dir)):
            if name.endswith(".tmp"):
                continue
            spec = deserialize_jobspec(os.path.join(self.active_job_dir, name))
            out[name] = BastionJob(spec=spec, state=self.get_job_state(name) or JobStatus(JobState.PENDING))
        return out


class Bastion(Configurable):
    @config_class
    class Config(Configurable.Config):
        root_dir: Required[str] = REQUIRED
        scheduler: Required[InstantiableConfig] = REQUIRED
        cleaner: Optional[InstantiableConfig] = None
        update_interval_seconds: float = 30.0
        # Seconds a pre-empted or cancelled command gets between SIGTERM and SIGKILL.
        termination_grace_seconds: float = 10.0
        # Publish a lifecycle event per job state change to ``<root_dir>/events.jsonl``.
        publish_events: bool = False
        # Where elastic jobs' desired replica counts come from and granted counts go to
        # (``cloud.common.replica_manager``); None: elastic jobs run at their minimum.
        replica_manager: Optional[InstantiableConfig] = None

    def __init__(self, cfg):
        super().__init__(cfg)
        self._event_client = None
        self._published: dict[str, str] = {}
        if cfg.publish_events:
            from axlearn_b200.cloud.common.event_queue import FileQueueClient

            self._event_client = FileQueueClient(os.path.join(cfg.root_dir, "events.jsonl"))
        self._dir = BastionDirectory.default_config().set(root_dir=cfg.root_dir).instantiate()
        self._scheduler: JobScheduler = cfg.scheduler.instantiate()
        self._cleaner = cfg.cleaner.instantiate() if cfg.cleaner is not None else None
        self._replica_manager = cfg.replica_manager.instantiate() if cfg.replica_manager is not None else None
        self._jobs: dict[str, BastionJob] = {}

    @property
    def directory(self) -> BastionDirectory:
        return self._dir

    # ------------------------------------------------------------------ processes
    def _start(self, job: BastionJob, command: str, log_name: str) -> _Running:
        log = open(os.path.join(self._dir.logs_dir, log_name), "a", encoding="utf-8")  # pylint: disable=consider-using-with
        env = dict(os.environ)
        env.update({k: str(v) for k, v in (job.spec.env_vars or {}).items()})
        env["BASTION_JOB_NAME"] = job.spec.name
        if "tier" in job.state.metadata:
            env["BASTION_TIER"] = str(job.state.metadata["tier"])
        proc = subprocess.Popen(shlex.split(command), stdout=log, stderr=subprocess.STDOUT, env=env,  # pylint: disable=consider-using-with
                                start_new_session=True)
        return _Running(proc, log)

    def _stop(self, running: Optional[_Running]) -> None:
        if running is None:
            return
        proc = running.process
        if proc.poll() is None:
            try:
                os.killpg(proc.pid, signal.SIGTERM)   # the job's own process group, by exact id
            except ProcessLookupError:
                pass
            try:
                proc.wait(timeout=self._config.termination_grace_seconds)
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(proc.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
                proc.wait()
        running.log.close()

    # ------------------------------------------------------------------ one pass
    def _sync_jobs(self) -> None:
        on_disk = self._dir.list_jobs()
        for name, job in on_disk.items():
            if name not in self._jobs:
                # A job found ACTIVE on disk belongs to an earlier bastion process: its command
                # is gone, so it starts over from PENDING (and resumes from its checkpoints).
                state = job.state
                if state.state == JobState.ACTIVE:
                    state = JobStatus(JobState.PENDING)
                self._jobs[name] = BastionJob(spec=job.spec, state=state)
        for name in list(self._jobs):
            if name not in on_disk:
                self._stop(self._jobs[name].command_proc)
                del self._jobs[name]
        for name, job in self._jobs.items():
            user_state = os.path.join(self._dir.user_states_dir, name)
            if os.path.exists(user_state) and job.state.state in (JobState.PENDING, JobState.ACTIVE):
                job.state = JobStatus(JobState.CANCELLING)

    def _write_state(self, name: str, job: BastionJob) -> None:
        path = os.path.join(self._dir.job_states_dir, name)
        with open(path + ".tmp", "w", encoding="utf-8") as f:
            json.dump({"state": job.state.state.value, "metadata": job.state.metadata}, f)
        os.replace(path + ".tmp", path)

    def _complete(self, name: str) -> None:
        src = os.path.join(self._dir.active_job_dir, name)
        if os.path.exists(src):
            os.replace(src, os.path.join(self._dir.complete_job_dir, name))
        user_state = os.path.join(self._dir.user_states_dir, name)
        if os.path.exists(user_state):
            os.remove(user_state)

    def execute_once(self) -> dict[str, JobStatus]:
        self._sync_jobs()
        # 1. Collect what finished; move cancelled jobs on.
        for name, job in self._jobs.items():
            st = job.state.state
            if st == JobState.ACTIVE and job.command_proc is not None and job.command_proc.process.poll() is not None:
                rc = job.command_proc.process.returncode
                job.command_proc.log.close()
                job.command_proc = None
                job.state = JobStatus(JobState.CLEANING, {"returncode": rc})
            elif st == JobState.CANCELLING:
                self._stop(job.command_proc)
                job.command_proc = None
                job.state = JobStatus(JobState.CLEANING, {"cancelled": True})
            if job.state.state == JobState.CLEANING:
                if job.cleanup_proc is None and job.spec.cleanup_command and not job.state.metadata.get("cleanup_started"):
                    job.cleanup_proc = self._start(job, job.spec.cleanup_command, f"{name}.cleanup")
                    job.state.metadata["cleanup_started"] = True
                if job.cleanup_proc is None or job.cleanup_proc.process.poll() is not None:
                    if job.cleanup_proc is not None:
                        job.cleanup_proc.log.close()
                        job.cleanup_proc = None
                    job.state = JobStatus(JobState.COMPLETED, job.state.metadata)
        # 2. Schedule the schedulable ones.
        candidates = {n: j.spec.metadata for n, j in self._jobs.items()
                      if j.state.state in (JobState.PENDING, JobState.ACTIVE)}
        desired = {}
        if self._replica_manager is not None:
            self._replica_manager.refresh()
            for n, meta in candidates.items():
                if getattr(meta, "scaling_specs", None):
                    want = self._replica_manager.get_desired_replicas(n)
                    if want:
                        desired[n] = want
        verdicts = self._scheduler.schedule(candidates, desired_replicas=desired).job_verdicts if candidates else {}
        for name, verdict in verdicts.items():
            job = self._jobs[name]
            if self._replica_manager is not None and verdict and "granted_replicas" in verdict.metadata:
                self._replica_manager.set_granted_replicas(name, verdict.metadata["granted_replicas"])
            if verdict and job.state.state == JobState.PENDING:
                job.state = JobStatus(JobState.ACTIVE, dict(verdict.metadata))
                job.command_proc = self._start(job, job.spec.command, name)
            elif not verdict and job.state.state == JobState.ACTIVE:
                logging.info("pre-empting %s: over limits on %s", name, verdict.over_limits)
                self._stop(job.command_proc)
                job.command_proc = None
                job.state = JobStatus(JobState.PENDING, {"preempted": True})
            elif verdict and job.state.state == JobState.ACTIVE:
                job.state.metadata.update(verdict.metadata)
        # 3. Jobs that can never run are cancelled by the cleaner.
        if self._cleaner is not None:
            pending = {n: j.spec for n, j in self._jobs.items() if j.state.state == JobState.PENDING}
            for name in self._cleaner.sweep(pending):
                self._jobs[name].state = JobStatus(JobState.COMPLETED, {"unschedulable": True})
        # 4. Persist.
        for name, job in list(self._jobs.items()):
            self._write_state(name, job)
            if self._event_client is not None and self._published.get(name) != job.state.state.value:
                from axlearn_b200.cloud.common.event_queue import JobLifecycleEvent

                self._published[name] = job.state.state.value
                self._event_client.publish(JobLifecycleEvent(
                    job_name=name, state=job.state.state.value, details=json.dumps(job.state.metadata or {}, default=str)))
            if job.state.state == JobState.COMPLETED:
                self._complete(name)
                del self._jobs[name]
        return {n: j.state for n, j in self._jobs.items()}

    def execute(self, *, max_iterations: Optional[int] = None) -> None:
        i = 0
        try:
            while max_iterations is None or i < max_iterations:
                start = time.time()
                self.execute_once()
                i += 1
                left = self._config.update_interval_seconds - (time.time() - start)
                if left > 0 and (max_iterations is None or i < max_iterations):
                    time.sleep(left)
        finally:
            self.shutdown()

    def shutdown(self) -> None:
        for job in self._jobs.values():
            self._stop(job.command_proc)
            self._stop(job.cleanup_proc)
            job.command_proc = job.cleanup_proc = None
