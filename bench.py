"""Headline benchmark: Fuji-7B training throughput (tokens/s) on N B200 GPUs of one node.

Config (the reference's single-host Fuji-7B-v2 training configuration): 32 layers, d_model 4096, 32 heads (MHA), SwiGLU hidden 11008,
vocab 32768, RoPE, RMSNorm; sequence length 4096; 4 sequences per GPU (32 at 8 GPUs, weak
scaling); mesh fsdp=N; bf16 compute with fp32 master weights and AdamW moments; full
rematerialisation per layer; synthetic uniform-random tokens from seed 0; random-init weights.

Two measurements per run:
  * ``value``: K steps of the trainer's step function on device-resident batches, timed with
    CUDA events between barriers, max over ranks.
  * ``e2e``: the same K steps through the public ``SpmdTrainer.train_step(host_batch)`` with a
    pinned-host → device copy of every batch and a device → host read of every loss.

``--impl reference`` would run the unmodified reference (apple/axlearn, JAX/XLA); it cannot be
installed offline here (no ``hatchling`` build backend, no ``jax``/``jaxlib``/``tensorstore``
wheels), so that arm reports ``unavailable``.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

PUBLISHED_TOKENS_PER_S = 65536 / 1.54  # fuji-7B-v2 single host, 8xH100 (fuji.py:1214-1216)


def _args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="7B", help="Fuji size (7B is the benchmark; others for debugging), or an "
                    "envy preset with --family envy (Mixtral-8x7B: the MoE training configuration)")
    ap.add_argument("--family", default="fuji", choices=["fuji", "envy"])
    ap.add_argument("--drop_free", action="store_true", help="--family envy: capacity-free routing on the grouped GEMM "
                    "(TransformerFeedForwardDropFreeMoE) instead of the capacity-based layer")
    ap.add_argument("--ep_capacity", type=float, default=None, help="--drop_free with an expert axis: cap every rank's row "
                    "buffer at this multiple of the fair share (default: sized for the worst case, nothing dropped)")
    ap.add_argument("--tp_seq", action="store_true", help="non-headline, with a model axis in --mesh: sequence-sharded "
                    "norm / residual regions (all-gather into column-parallel, reduce-scatter out of row-parallel linears)")
    ap.add_argument("--fp8", action="store_true", help="block-scaled fp8 projection GEMMs (FP8ConfigModifier)")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--per_gpu_batch", type=int, default=4)
    ap.add_argument("--layers", type=int, default=None, help="debug only: override layer count")
    ap.add_argument("--skip_e2e", action="store_true")
    ap.add_argument("--mesh", default=None, help="non-headline: mesh axes instead of fsdp=N, e.g. 'fsdp=4,model=2' "
                    "(the product of the sizes must be --gpus; the batch is per data-parallel rank)")
    ap.add_argument("--kernel_table", default=None, help="after the timed regions, profile two more steps with the "
                    "torch profiler and write per-kernel device-time shares to this file (rank 0)")
    ap.add_argument("--skip_parity", action="store_true", help="N>1: skip the one-step fused-vs-library parity record")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self._idx = gpu_index
        self._proc = None
        self._lines: list[str] = []
        self._thread = None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self._idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self):
        for line in self._proc.stdout:
            self._lines.append(line.strip())

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self._lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def main():
    args = _args()
    if args.impl == "reference":
        print(json.dumps({
            "impl": "reference",
            "unavailable": "apple/axlearn needs jax/jaxlib(cuda12)/tensorstore/optax wheels and the hatchling "
                           "build backend; none are in the offline wheelhouse, so it cannot be installed",
        }))
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()  # CPU is only for dry-running this script's plumbing.
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # Collectives share the GPU with persistent compute kernels: cap their CTA count.
        os.environ.setdefault("NCCL_MAX_CTAS", os.environ.get("AXB200_COMM_SMS", "16"))
        if use_cuda:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        else:
            dist.init_process_group("gloo")
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    from axlearn_b200.ops import cuda_ops

    moe = args.family == "envy"
    parity = None
    if world > 1 and use_cuda and not moe and not args.skip_parity and not args.mesh:
        parity = _fused_vs_library_parity(args, world, local_rank)
    trainer, mk = _build_trainer(args, world, local_rank, use_cuda, layers=args.layers, per_gpu_batch=args.per_gpu_batch)
    global_batch = args.per_gpu_batch * _data_ranks(args, world, moe)
    num_params = sum(t.numel() for t in _leaves(trainer.trainer_state["model"]))
    data = iter(trainer.input.dataset())
    dev = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")

    def barrier():
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    class _WallEvent:
        def __init__(self, enable_timing=True):
            self.t = 0.0

        def record(self):
            self.t = time.perf_counter()

        def elapsed_time(self, other):
            return (other.t - self.t) * 1e3

    Event = torch.cuda.Event if use_cuda else _WallEvent

    tokens_per_step = global_batch * args.seq

    # ----------------------------------------------------------------- device-timed region
    device_batches = [
        {k: v.to(dev) for k, v in next(data).items()} for _ in range(min(4, args.warmup + args.steps))]
    step_fn = trainer._train_step  # pylint: disable=protected-access
    with trainer.mesh():
        for i in range(args.warmup):
            out = step_fn(device_batches[i % len(device_batches)])
        barrier()
        if use_cuda:
            cuda_ops.check_status()
        sampler = ClockSampler(local_rank)
        sampler.start()
        launches0 = cuda_ops.launch_count
        start, end = Event(enable_timing=True), Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(args.steps):
            out = step_fn(device_batches[(args.warmup + i) % len(device_batches)])
        end.record()
        barrier()
        clocks = sampler.stop()
        launches = cuda_ops.launch_count - launches0
        ms = start.elapsed_time(end)
    loss_value = float(out["loss"])
    if use_cuda:
        cuda_ops.check_status()
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)

    # ----------------------------------------------------------------- end-to-end region
    e2e = None
    if not args.skip_e2e:
        host_batches = [next(data) for _ in range(args.steps)]
        h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values())
        barrier()
        t0 = time.perf_counter()
        for hb in host_batches:
            out = trainer.train_step(hb)
            _ = out["loss"].item()  # device -> host read of the step's result
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {
            "value": tokens_per_step * args.steps / dt.item(), "unit": "tokens/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
        }

    if args.kernel_table and use_cuda:
        _write_kernel_table(args.kernel_table, trainer, step_fn, device_batches, rank)

    if rank == 0:
        # 6 * params * tokens (fwd+bwd) + attention; remat adds one more forward (reported
        # MFU counts model FLOPs only, i.e. without the recompute).
        layers, d, heads = mk["num_layers"], mk["hidden_dim"], mk["num_heads"]
        if moe:
            kvd = d * mk["num_kv_heads"] // heads
            # Active parameters per token: attention + 2 of the experts.
            dense_params = layers * (2 * d * d + 2 * d * kvd + 2 * 3 * d * mk["moe_ffn_dim"]) + mk["vocab_size"] * d
        else:
            dense_params = layers * (4 * d * d + 3 * d * 11008) + 32768 * d
        flops_per_token = 6 * dense_params + 6 * layers * d * args.seq  # causal attention: 12*L*d*T/2
        peak = 2.25e15
        result = {
            "metric": ("MoE train tokens/sec (max over ranks)" if moe else "Fuji-7B train tokens/sec (max over ranks)"),
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None if moe else value / PUBLISHED_TOKENS_PER_S, "dtype": "fp8 (block-scaled projections) + bf16" if args.fp8 else "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {
                "model": (f"envy-{args.model}" if moe else f"fuji-{args.model}-v2") + (
                    f"-{args.layers}layers-DEBUG" if args.layers else "") + ("-dropfree" if args.drop_free else ""),
                "global_batch": global_batch, "seq_len": args.seq,
                "parallelism": (args.mesh.replace("=", "").replace(",", "x") + " (non-headline mesh)") if args.mesh else (
                    f"expert{world} (dense parameters sharded over the same axis)" if moe else f"fsdp{world}"),
                "remat": "full per layer", "optimizer": "clip_by_global_norm(1)+adamw_decoupled, fp32 master+moments",
                "l2": "per-step working set (>100 GB of parameters, moments and activations) exceeds the 126 MB L2",
            },
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": launches,
            "multi_gpu_parity": parity,
            "loss": loss_value,
            "mfu_model_flops_nominal_peak": value * flops_per_token / (peak * world),
            "local_params": num_params,
        }
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


def _build_trainer(args, world, local_rank, use_cuda, *, layers, per_gpu_batch):
    """The benchmark's trainer (optionally a slice with fewer layers); returns (trainer, model kwargs)."""
    import torch

    from axlearn_b200.common import prng
    from axlearn_b200.common.base_layer import RematSpec, nothing_saveable
    from axlearn_b200.experiments.text.gpt import fuji
    from axlearn_b200.experiments.text.gpt.common import (
        MESH_AXIS_NAMES,
        adamw_decoupled_learner_config,
        get_trainer_config_fn,
        mesh_shape_from_axes,
    )

    moe = args.family == "envy"
    kw = fuji.get_trainer_kwargs("7B" if moe else args.model, vocab_size=32768, version=fuji.Version.V2)
    if moe:
        from axlearn_b200.experiments.text.gpt import envy

        mk = dict(envy.MODEL_PRESETS[args.model])
        if layers:
            mk["num_layers"] = layers
        if args.drop_free:
            mk["drop_free"] = True
        model_cfg = envy.model_config(scan_chunk=8192, **mk)
        if args.drop_free and args.ep_capacity is not None:
            ff = model_cfg.decoder.transformer.layer.feed_forward
            if "expert_parallel_capacity" in ff.keys():
                ff.expert_parallel_capacity = args.ep_capacity
    else:
        mk = dict(kw["model_kwargs"])
        if layers:
            mk["num_layers"] = layers
        model_cfg = fuji.model_config(scan_chunk=8192, **mk)
    # Full remat per layer: only each layer's input is kept.
    model_cfg.decoder.transformer.layer.remat_spec = RematSpec(prevent_cse=False, policy=nothing_saveable)
    if args.tp_seq:
        model_cfg.decoder.transformer.tp_sequence_parallel = True
    cfg = get_trainer_config_fn(
        model_cfg=model_cfg,
        learner_cfg=adamw_decoupled_learner_config(max_step=kw["max_step"], **kw["learner_kwargs"]),
        max_step=kw["max_step"], train_batch_size=per_gpu_batch * _data_ranks(args, world, moe),
        max_sequence_length=args.seq,
        vocab_size=mk.get("vocab_size", 32768),
        mesh_shape=mesh_shape_from_axes(**_mesh_axes(args, world, moe)),
        mesh_axis_names=MESH_AXIS_NAMES,
        train_dtype=torch.bfloat16)()
    if args.fp8:
        from axlearn_b200.common.trainer_config_modifier import FP8ConfigModifier

        cfg = FP8ConfigModifier.default_config().set(scaling="block").instantiate()(cfg)
    cfg.dir = tempfile.mkdtemp(prefix="axb200_bench_")
    cfg.device = f"cuda:{local_rank}" if use_cuda else "cpu"
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    return trainer, mk


def _mesh_axes(args, world: int, moe: bool) -> dict:
    if args.mesh:
        axes = {k: int(v) for k, v in (item.split("=") for item in args.mesh.split(","))}
        size = 1
        for v in axes.values():
            size *= v
        assert size == world, f"--mesh {args.mesh} has {size} ranks but --gpus is {world}"
        return axes
    return {"expert": world} if moe else {"fsdp": world}


def _data_ranks(args, world: int, moe: bool) -> int:
    """Ranks that hold different data (everything but the model / pipeline / seq axes)."""
    axes = _mesh_axes(args, world, moe)
    n = 1
    for k, v in axes.items():
        if k in ("data", "expert", "fsdp"):
            n *= v
    return n


def _fused_vs_library_parity(args, world, local_rank) -> dict:
    """Multi-GPU correctness record carried by the benchmark line: a 2-layer slice of the same
    architecture (same widths, sequence length and mesh) takes ONE training step from the same
    initial state and batch, first with library collectives (all-gather / reduce-scatter through
    NCCL), then with the fused gather-GEMM / GEMM-reduce-scatter kernels; reports both losses and
    the largest gradient-shard difference relative to the largest gradient, max over ranks."""
    import gc

    import torch
    import torch.distributed as dist

    from axlearn_b200.common.utils import flatten_items
    from axlearn_b200.ops import cuda_ops
    from axlearn_b200.parallel import fsdp_fused

    was_enabled = fsdp_fused.ENABLED
    record = {}
    grads = {}
    for name, fused in (("library", False), ("fused", True)):
        fsdp_fused.ENABLED = fused and was_enabled
        fsdp_fused.reset()
        trainer, _ = _build_trainer(args, world, local_rank, True, layers=2, per_gpu_batch=1)
        out = trainer.train_step(next(iter(trainer.input.dataset())))
        record[f"loss_{name}"] = float(out["loss"])
        stacked = trainer._shadows["decoder"]["transformer"]["repeat"]["layer"]  # pylint: disable=protected-access
        grads[name] = {p: t.grad.float().clone() for p, t in flatten_items(stacked) if t.grad is not None}
        torch.cuda.synchronize()
        cuda_ops.check_status()
        del trainer, out, stacked
        fsdp_fused.reset()
        gc.collect()
        torch.cuda.empty_cache()
    fsdp_fused.ENABLED = was_enabled
    worst = torch.zeros(2, device="cuda")
    for p, g in grads["fused"].items():
        r = grads["library"][p]
        worst[0] = torch.maximum(worst[0], (g - r).abs().max())
        worst[1] = torch.maximum(worst[1], r.abs().max())
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    record["max_grad_shard_abs_diff"] = worst[0].item()
    record["max_grad_abs"] = worst[1].item()
    record["max_grad_shard_rel_diff"] = worst[0].item() / max(worst[1].item(), 1e-30)
    record["fused_path_active"] = bool(was_enabled)
    record["slice"] = f"2 layers of the benchmark architecture, 1x{args.seq} tokens per GPU, fsdp{world}, one step"
    del grads
    gc.collect()
    torch.cuda.empty_cache()
    return record


def _write_kernel_table(path, trainer, step_fn, batches, rank) -> None:
    """Device time per kernel over two profiled steps (outside every timed region)."""
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    with trainer.mesh():
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(2):
                step_fn(batches[i % len(batches)])
            torch.cuda.synchronize()
    total, count = collections.Counter(), collections.Counter()
    first = last = None
    for e in prof.events():
        if e.device_type != torch.autograd.DeviceType.CUDA:
            continue
        total[e.name[:100]] += e.device_time
        count[e.name[:100]] += 1
        first = e.time_range.start if first is None else min(first, e.time_range.start)
        last = e.time_range.end if last is None else max(last, e.time_range.end)
    if rank != 0 or not total:
        return
    busy = sum(total.values())
    with open(path, "w", encoding="utf-8") as f:
        f.write(f"span_ms_per_step {(last - first) / 2e3:.1f} busy_ms_per_step {busy / 2e3:.1f} "
                f"launches_per_step {sum(count.values()) // 2}\n")
        for name, t in total.most_common(40):
            f.write(f"{100 * t / busy:5.1f}% {count[name] // 2:5d} {t / count[name]:9.1f}us  {name}\n")


def _leaves(tree):
    if isinstance(tree, dict):
        for v in tree.values():
            yield from _leaves(v)
    elif tree is not None and hasattr(tree, "numel"):
        yield tree


if __name__ == "__main__":
    main()
