"""Argument parsing and dispatch of the command tree (see the package docstring)."""

from __future__ import annotations

import argparse
import datetime
import getpass
import json
import os
import subprocess
import sys
from typing import Optional, Sequence


def _bastion_scheduler_cfg(quota_file: str):
    from axlearn_b200.cloud.common import quota
    from axlearn_b200.cloud.common.scheduler import JobScheduler
    from axlearn_b200.common.config import config_for_function

    return JobScheduler.default_config().set(quota=config_for_function(quota.get_resource_limits).set(path=quota_file))


def _cmd_bastion(args) -> int:
    from axlearn_b200.cloud.common.bastion import Bastion, BastionDirectory
    from axlearn_b200.cloud.common.cleaner import UnschedulableCleaner
    from axlearn_b200.cloud.common.job_types import JobMetadata, JobSpec

    directory = BastionDirectory.default_config().set(root_dir=args.root_dir).instantiate()
    if args.action == "start":
        sched = _bastion_scheduler_cfg(args.quota_file)
        cfg = Bastion.default_config().set(
            root_dir=args.root_dir, scheduler=sched, update_interval_seconds=args.interval,
            cleaner=UnschedulableCleaner.default_config().set(scheduler=sched))
        cfg.instantiate().execute(max_iterations=args.max_iterations)
        return 0
    if args.action == "submit":
        resources = dict((k, int(v)) for k, v in (item.split("=") for item in args.resources))
        meta = JobMetadata(user_id=args.user or getpass.getuser(), project_id=args.project,
                           creation_time=datetime.datetime.now(), resources=resources, priority=args.priority,
                           job_id=args.name)
        env = dict(item.split("=", 1) for item in args.env)
        directory.submit_job(args.name, job_spec=JobSpec(
            version=1, name=args.name, command=args.command, cleanup_command=args.cleanup_command, env_vars=env,
            metadata=meta))
        print(f"submitted {args.name}")
        return 0
    if args.action == "cancel":
        directory.cancel_job(args.name)
        print(f"cancelling {args.name}")
        return 0
    if args.action == "state":
        st = directory.get_job_state(args.name)
        print(json.dumps(None if st is None else {"state": st.state.value, "metadata": st.metadata}))
        return 0
    rows = [{"name": n, "state": j.state.state.value, "user": j.spec.metadata.user_id,
             "project": j.spec.metadata.project_id, "resources": j.spec.metadata.resources}
            for n, j in directory.list_jobs().items()]
    print(json.dumps(rows, indent=1))
    return 0


def _cmd_bundle(args) -> int:
    from axlearn_b200.cloud.common.bundler import get_bundler_config

    cfg = get_bundler_config(bundler_type="tar", spec=[f"remote_dir={args.remote_dir}"] + list(args.spec))
    print(cfg.instantiate().bundle(args.name, src_dir=args.src_dir))
    return 0


def _cmd_train(args, rest: Sequence[str]) -> int:
    cmd = [sys.executable, "-m", "axlearn_b200.common.launch_trainer_main", *rest]
    if args.gpus > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "-m", "axlearn_b200.common.launch_trainer_main", *rest]
    return subprocess.call(cmd)


def _cmd_bench(args, rest: Sequence[str]) -> int:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    return subprocess.call([sys.executable, os.path.join(root, "bench.py"), *rest])


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="axlearn_b200")
    groups = ap.add_subparsers(dest="group", required=True)

    train = groups.add_parser("train", help="run a trainer config; unknown flags go to launch_trainer_main")
    train.add_argument("--gpus", type=int, default=1)
    groups.add_parser("bench", help="run bench.py; flags are passed through")

    bastion = groups.add_parser("bastion")
    bastion.add_argument("action", choices=["start", "submit", "cancel", "list", "state"])
    bastion.add_argument("--root_dir", required=True)
    bastion.add_argument("--quota_file")
    bastion.add_argument("--interval", type=float, default=30.0)
    bastion.add_argument("--max_iterations", type=int, default=None)
    bastion.add_argument("--name")
    bastion.add_argument("--command")
    bastion.add_argument("--cleanup_command")
    bastion.add_argument("--project", default="default")
    bastion.add_argument("--user")
    bastion.add_argument("--priority", type=int, default=5)
    bastion.add_argument("--resources", nargs="*", default=[], help="e.g. b200=8")
    bastion.add_argument("--env", nargs="*", default=[], help="KEY=VALUE")

    bundle = groups.add_parser("bundle")
    bundle.add_argument("--name", required=True)
    bundle.add_argument("--remote_dir", required=True)
    bundle.add_argument("--src_dir", default=".")
    bundle.add_argument("--spec", nargs="*", default=[])
    return ap


def main(argv: Optional[Sequence[str]] = None) -> int:
    args, rest = build_parser().parse_known_args(argv)
    if args.group == "train":
        return _cmd_train(args, rest)
    if args.group == "bench":
        return _cmd_bench(args, rest)
    if rest:
        raise SystemExit(f"unknown arguments: {rest}")
    if args.group == "bastion":
        if args.action == "start" and not args.quota_file:
            raise SystemExit("bastion start needs --quota_file")
        if args.action in ("submit", "cancel", "state") and not args.name:
            raise SystemExit(f"bastion {args.action} needs --name")
        if args.action == "submit" and not args.command:
            raise SystemExit("bastion submit needs --command")
        return _cmd_bastion(args)
    return _cmd_bundle(args)
