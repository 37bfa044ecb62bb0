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
    if args.format == "table":
        from axlearn_b200.cloud.common import utils as cloud_utils

        jobs = directory.list_jobs()
        print(cloud_utils.jobs_table(jobs))
        print("Usage by project:", cloud_utils.project_usage_table(jobs))
        print("Usage by user:", cloud_utils.user_usage_table(jobs))
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


def _cmd_gcp(args, rest: Sequence[str]) -> int:
    """``gcp launch|delete|status|manifest|config``: GKE JobSets through kubectl, settings from the
    ``[gcp]`` tables of the settings files (axlearn/cloud/gcp/jobs/launch.py, .../config.py)."""
    from axlearn_b200.cloud.common import config as settings
    from axlearn_b200.cloud.gcp.job import GKEJob
    from axlearn_b200.cloud.gcp.jobset_utils import A3UltraReplicatedJob, A4HighReplicatedJob, GCSFuseMount

    if args.action == "config":
        if args.activate:
            _, gcp = settings.load_configs("gcp")
            if args.activate not in gcp:
                raise SystemExit(f"no [gcp.\"{args.activate}\"] table; known: {[k for k in gcp if k != '_active']}")
            gcp["_active"] = args.activate
            print(settings.update_configs("gcp", gcp))
        else:
            path, gcp = settings.load_configs("gcp")
            print(json.dumps({"file": path, "gcp": gcp}, indent=1))
        return 0
    if not args.name:
        raise SystemExit(f"gcp {args.action} needs --name")

    def setting(key, default=None, required=False):
        return settings.gcp_settings(key, project=args.project, env_id=args.env_id, default=default, required=required)

    if rest and rest[0] == "--":
        rest = rest[1:]          # the separator in front of the worker command is not part of it
    command = " ".join(rest) if rest else (args.command or "true")
    if args.action == "logs":
        # Direct route: the cluster's own log stream.  (Cloud Logging: ``cloud.gcp.logs.print_logs``
        # with an authorised client.)
        from axlearn_b200.cloud.gcp import logs  # pylint: disable=import-outside-toplevel

        cmd = list(logs.kubectl_logs_command(name=args.name, worker=args.worker, replica=args.replica,
                                             namespace=args.namespace, num_lines=args.num_lines, follow=args.follow))
        print(" ".join(cmd))
        print("Cloud logging url: " + logs.logs_url(name=args.name, worker=args.worker, replica=args.replica,
                                                     namespace=args.namespace))
        if args.dry_run:
            return 0
        import subprocess  # pylint: disable=import-outside-toplevel

        return subprocess.run(cmd, check=False).returncode
    if args.action == "serve-manifest":
        # A multi-host serving deployment: --num_nodes hosts per replica, leader Service, probes,
        # optionally a Gateway route and an autoscaler (axlearn/cloud/gcp/lws_utils.py, k8s_*.py).
        import yaml  # pylint: disable=import-outside-toplevel

        from axlearn_b200.cloud.gcp import serving

        lws = serving.LeaderWorkerSet.default_config().set(
            name=args.name, namespace=args.namespace, image=args.image or setting("docker_image", required=True),
            command=command, replicas=args.replicas, hosts_per_replica=args.num_nodes, machine_type=args.machine_type,
            service_account=setting("k8s_service_account"), port=args.port,
            env_vars=dict(item.split("=", 1) for item in args.env),
            probes=[serving.StartupProbe.default_config().set(port=args.port),
                    serving.ReadinessProbe.default_config().set(port=args.port),
                    serving.LivenessProbe.default_config().set(port=args.port)])
        dep = serving.ServingDeployment.default_config().set(lws=lws, gke_policies=bool(args.gateway),
                                                             monitoring=args.max_replicas > args.replicas)
        if args.gateway:
            dep.route = serving.LWSHTTPRoute.default_config().set(gateway_name=args.gateway)
        if args.max_replicas > args.replicas:
            metric, _, target = args.scale_metric.partition("=")
            dep.hpa = serving.HPA.default_config().set(
                min_replicas=args.replicas, max_replicas=args.max_replicas,
                metrics=[serving.HPAMetric.default_config().set(metric_name=metric, average_value=target or "1")])
        objs = [lws.instantiate().build()] + dep.instantiate().manifests()
        print(yaml.safe_dump_all(objs, sort_keys=False))
        return 0
    builder_cls = {"a4-highgpu-8g": A4HighReplicatedJob, "a3-ultragpu-8g": A3UltraReplicatedJob}[args.machine_type]
    builder = builder_cls.default_config().set(
        command=command, image=args.image or setting("docker_image"), num_nodes=args.num_nodes,
        reservation=args.reservation or setting("reservation"), service_account=setting("k8s_service_account"),
        priority_class=args.priority_class, disable_nvls=args.fault_tolerant,
        env_vars=dict(item.split("=", 1) for item in args.env))
    if args.output_dir and args.output_dir.startswith("gs://"):
        builder.gcsfuse_mount = GCSFuseMount(gcs_path=args.output_dir)
        builder.output_dir = "/output"
    job = GKEJob.default_config().set(name=args.name, builder=builder, namespace=args.namespace,
                                      max_restarts=args.max_tries - 1, queue=setting("kueue_queue")).instantiate()
    if args.action == "manifest":
        import yaml  # pylint: disable=import-outside-toplevel

        print(yaml.safe_dump(job.build_jobset(), sort_keys=False))
    elif args.action == "launch":
        print(job.execute())
    elif args.action == "delete":
        job._delete()  # pylint: disable=protected-access
        print(f"deleted {args.name}")
    else:
        print(job.status().value)
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
    bastion.add_argument("--format", default="json", choices=["json", "table"], help="list: output form")

    gcp = groups.add_parser("gcp", help="GKE JobSets; everything after the flags is the worker command")
    gcp.add_argument("action", choices=["launch", "delete", "status", "manifest", "config", "serve-manifest", "logs"])
    gcp.add_argument("--worker", type=int, default=0, help="logs: worker (completion index) within the replica")
    gcp.add_argument("--replica", type=int, default=0, help="logs: replicated-job index")
    gcp.add_argument("--num_lines", "-n", type=int, default=1000, help="logs: lines to show")
    gcp.add_argument("--follow", action="store_true", help="logs: keep streaming")
    gcp.add_argument("--dry_run", action="store_true", help="logs: print the command and the URL only")
    gcp.add_argument("--name")
    gcp.add_argument("--project")
    gcp.add_argument("--env_id")
    gcp.add_argument("--namespace", default="default")
    gcp.add_argument("--machine_type", default="a4-highgpu-8g", choices=["a4-highgpu-8g", "a3-ultragpu-8g"])
    gcp.add_argument("--num_nodes", type=int, default=1)
    gcp.add_argument("--image")
    gcp.add_argument("--command")
    gcp.add_argument("--reservation")
    gcp.add_argument("--priority_class")
    gcp.add_argument("--output_dir")
    gcp.add_argument("--max_tries", type=int, default=1)
    gcp.add_argument("--fault_tolerant", action="store_true", help="restartable job: no NVLink multicast binding")
    gcp.add_argument("--env", nargs="*", default=[], help="KEY=VALUE")
    gcp.add_argument("--activate", help="config: make this \"project:env_id\" table the active one")
    gcp.add_argument("--replicas", type=int, default=1, help="serve-manifest: LeaderWorkerSet replicas")
    gcp.add_argument("--max_replicas", type=int, default=0, help="serve-manifest: > replicas adds an autoscaler")
    gcp.add_argument("--scale_metric", default="requests_in_flight=16",
                     help="serve-manifest: pod metric and its per-pod target for the autoscaler")
    gcp.add_argument("--port", type=int, default=8000, help="serve-manifest: the leader's HTTP port")
    gcp.add_argument("--gateway", help="serve-manifest: route requests from this Gateway to the deployment")

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
    if args.group == "gcp":
        return _cmd_gcp(args, rest)
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
