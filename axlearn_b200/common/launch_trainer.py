"""Builds and runs a trainer from a named config; the library half of ``launch_trainer_main``.

Parity targets in the reference: flags of ``launch_trainer`` (axlearn/common/launch_trainer.py:19-117:
``--module``, ``--config``, ``--trainer_dir``, ``--data_dir``, ``--mesh_selector``,
``--trainer_watchdog_timeout_seconds``, ``--trainer_crash_on_hang_timeout_seconds``,
``--trace_at_steps``), ``get_trainer_config`` (:120) and ``run_trainer`` (:150) which restores the
latest checkpoint (or initialises) and trains to ``max_step``.  absl flags become argparse.
"""

from __future__ import annotations

import argparse
import importlib
import json
import os
from typing import Any, Optional, Sequence

import torch

from axlearn_b200.common import prng


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Train a named config.")
    ap.add_argument("--module", required=True, help="module with named_trainer_configs(); "
                    "'text.gpt.c4_trainer' resolves under axlearn_b200.experiments")
    ap.add_argument("--config", required=True, help="name of the trainer config")
    ap.add_argument("--trainer_dir", required=True)
    ap.add_argument("--data_dir", default="FAKE")
    ap.add_argument("--mesh_selector", default=None)
    ap.add_argument("--max_step", type=int, default=None, help="override the config's max_step")
    ap.add_argument("--save_every_n_steps", type=int, default=None)
    ap.add_argument("--log_every_n_steps", type=int, default=None)
    ap.add_argument("--no_save_input_iterator", action="store_true",
                    help="do not checkpoint the input position (a resumed run then replays the data from the start)")
    ap.add_argument("--trainer_prng_seed", type=int, default=0)
    ap.add_argument("--trainer_watchdog_timeout_seconds", type=float, default=3600.0)
    ap.add_argument("--trainer_crash_on_hang_timeout_seconds", type=float, default=None)
    ap.add_argument("--trace_at_steps", default="", help="comma-separated steps at which to start a trace")
    ap.add_argument("--device", default=None, help="cpu | cuda[:N]; default: this rank's GPU if there is one")
    ap.add_argument("--status_port", type=int, default=None, help="serve thread stacks over HTTP on this port")
    ap.add_argument("--recorder_type", default=None, help="goodput recorder, e.g. 'file'")
    ap.add_argument("--recorder_spec", action="append", default=[], help="key=value for the recorder config "
                    "(repeatable); the 'file' recorder defaults to dir=<trainer_dir>/goodput")
    ap.add_argument("--distributed", action="store_true", help="join the torch.distributed job described by "
                    "RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT")
    return ap


def _import(module: str):
    for name in (module, f"axlearn_b200.experiments.{module}"):
        try:
            return importlib.import_module(name)
        except ModuleNotFoundError as e:
            if e.name not in (name, name.split(".")[0]) and not name.startswith(str(e.name)):
                raise
    raise ModuleNotFoundError(f"cannot import config module {module!r}")


def get_trainer_config(args: Any):
    mod = _import(args.module)
    configs = mod.named_trainer_configs()
    if args.config not in configs:
        from axlearn_b200.common.config import similar_names

        raise KeyError(f"unknown config {args.config!r}; did you mean {similar_names(args.config, list(configs))}?")
    cfg = configs[args.config]()
    cfg.dir = args.trainer_dir
    if args.max_step is not None:
        cfg.max_step = args.max_step
    if args.save_every_n_steps is not None:
        cfg.checkpointer.save_policy.n = args.save_every_n_steps
    # Input positions are a few integers here, so resuming exactly where the data left off is the default.
    cfg.save_input_iterator = not args.no_save_input_iterator
    if args.log_every_n_steps is not None:
        cfg.log_every_n_steps = args.log_every_n_steps
    if args.device:
        cfg.device = args.device
    cfg.watchdog_timeout_seconds = args.trainer_watchdog_timeout_seconds
    cfg.crash_on_hang_timeout_seconds = args.trainer_crash_on_hang_timeout_seconds
    if getattr(args, "recorder_type", None):
        from axlearn_b200.common import measurement

        spec = list(args.recorder_spec)
        if args.recorder_type == "file" and not any(item.startswith("dir=") for item in spec):
            spec.append(f"dir={os.path.join(args.trainer_dir, 'goodput')}")
        cfg.recorder = measurement.get_recorder_config(args.recorder_type, spec)
    if args.trace_at_steps:
        cfg.start_trace_steps = [int(s) for s in args.trace_at_steps.split(",") if s]
    if args.mesh_selector and getattr(cfg, "mesh_rules", None):
        from axlearn_b200.parallel.mesh import select_mesh_rule

        rule = select_mesh_rule(args.mesh_selector, cfg.mesh_rules)
        if rule is not None:
            cfg = rule(cfg) if callable(rule) else cfg.set(mesh_shape=rule)
    return cfg


def run_trainer(cfg, *, seed: int = 0, flags: Optional[dict] = None) -> Optional[dict]:
    """Records what is about to run -- ``{dir}/trainer_config`` (the config's debug string) and
    ``{dir}/launch_trainer_flags`` (the launch flags as JSON), written by process 0 -- then
    instantiates the trainer and runs it (reference: axlearn/common/launch_trainer.py:192-217)."""
    trainer_dir = getattr(cfg, "dir", None)
    if trainer_dir and _process_index() == 0:
        os.makedirs(trainer_dir, exist_ok=True)
        with open(os.path.join(trainer_dir, "trainer_config"), "w", encoding="utf-8") as f:
            f.write(cfg.debug_string())
        with open(os.path.join(trainer_dir, "launch_trainer_flags"), "w", encoding="utf-8") as f:
            json.dump(flags or {}, f, default=str, sort_keys=True)
    trainer = cfg.instantiate(parent=None)
    return trainer.run(prng.PRNGKey(seed))


def _process_index() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def main(argv: Optional[Sequence[str]] = None) -> None:
    args = parser().parse_args(argv)
    server = None
    if args.distributed:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        backend = "nccl" if torch.cuda.is_available() and (args.device or "cuda").startswith("cuda") else "gloo"
        dist.init_process_group(backend)
    if args.status_port is not None:
        from axlearn_b200.common.status_server import StatusHTTPServer

        server = StatusHTTPServer(args.status_port)
        server.start()
    try:
        os.makedirs(args.trainer_dir, exist_ok=True)
        run_trainer(get_trainer_config(args), seed=args.trainer_prng_seed, flags=vars(args))
    finally:
        if server is not None:
            server.stop()
        if args.distributed:
            import torch.distributed as dist

            dist.destroy_process_group()
