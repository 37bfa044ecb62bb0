"""Planning a training job without the hardware: per-GPU memory by category for a trainer config
on a given number of GPUs.

Parity target in the reference: axlearn/common/aot_compilation.py and
axlearn/experiments/run_aot_compilation.py (compile the train step for a TPU topology that is not
attached and print XLA's memory / cost analysis).  There is no compiler here; what can be known
ahead of time is the state layout, so the plan is computed from the parameter specs and the mesh:

* fp32 master parameters and the optimizer's moments, sharded over every mesh axis named in the
  parameter's ``mesh_axes`` (storage and compute axes alike);
* bf16 compute shadows and gradients with the same sharding;
* the fused-FSDP working set: two full-size gather buffers per stacked matrix (one layer each)
  and the per-layer gradient staging slots of the reduce-scatter;
* activations under full per-layer remat: one ``[B, T, D]`` checkpoint per layer plus the
  working set of the layer being recomputed, and the chunked logits of the fused loss.

``python -m axlearn_b200.common.aot_compilation --module text.gpt.c4_trainer --config fuji-7B-v2
--num_gpus 8`` prints the table and whether it fits 180 GB.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import math
from typing import Any, Optional, Sequence

from axlearn_b200.common.utils import flatten_items
from axlearn_b200.parallel.mesh import infer_mesh_shape

GIB = float(1 << 30)


@dataclasses.dataclass
class MemoryPlan:
    num_gpus: int
    mesh: dict
    total_params: int
    local_params: float
    bytes_per_gpu: dict
    hbm_bytes: float

    @property
    def total_bytes(self) -> float:
        return sum(self.bytes_per_gpu.values())

    @property
    def fits(self) -> bool:
        return self.total_bytes <= 0.92 * self.hbm_bytes       # head-room for the allocator and NCCL

    def table(self) -> str:
        rows = [f"mesh {self.mesh} on {self.num_gpus} GPUs; {self.total_params / 1e9:.2f} B parameters, "
                f"{self.local_params / 1e9:.3f} B per GPU"]
        for k, v in self.bytes_per_gpu.items():
            rows.append(f"  {k:<34} {v / GIB:9.2f} GiB")
        rows.append(f"  {'total':<34} {self.total_bytes / GIB:9.2f} GiB of {self.hbm_bytes / GIB:.0f} GiB "
                    f"-> {'fits' if self.fits else 'DOES NOT FIT'}")
        return "\n".join(rows)


def _axis_names(entry: Any) -> tuple:
    if entry is None:
        return ()
    if isinstance(entry, str):
        return (entry,)
    name = getattr(entry, "name", None)            # ComputeAxis("expert")
    if isinstance(name, str):
        return (name,)
    return tuple(n for e in entry for n in _axis_names(e))


def _shard_fraction(spec, mesh: dict) -> float:
    axes = spec.mesh_axes or ()
    denom = 1
    for entry in axes:
        for name in _axis_names(entry):
            denom *= mesh.get(name, 1)
    return 1.0 / denom


def plan_training_memory(trainer_cfg, *, num_gpus: int, hbm_gb: float = 180.0, moment_count: int = 2,
                         per_gpu_batch: Optional[int] = None, seq_len: Optional[int] = None) -> MemoryPlan:
    """``trainer_cfg``: an ``SpmdTrainer.Config``.  ``moment_count``: fp32 optimizer tensors per
    parameter (2 for Adam-style optimizers)."""
    names = tuple(trainer_cfg.mesh_axis_names)
    shape = infer_mesh_shape(tuple(trainer_cfg.mesh_shape), num_devices=num_gpus)
    mesh = dict(zip(names, shape))
    model = trainer_cfg.model.clone(name="model").instantiate(parent=None)
    specs = flatten_items(model.create_parameter_specs_recursively(), is_leaf=lambda x: hasattr(x, "mesh_axes"))
    total = sum(math.prod(s.shape) for _, s in specs)
    local = sum(math.prod(s.shape) * _shard_fraction(s, mesh) for _, s in specs)
    bf16 = trainer_cfg.train_dtype is not None and "bfloat16" in str(trainer_cfg.train_dtype)
    act_bytes = 2 if bf16 else 4
    out = {
        "fp32 master parameters": 4.0 * local,
        f"optimizer moments (x{moment_count}, fp32)": 4.0 * moment_count * local,
    }
    if bf16:
        out["bf16 compute copies"] = 2.0 * local
    out["gradients"] = float(act_bytes) * local
    # Fused FSDP: matrices that are stacked over layers and sharded over storage axes are gathered one
    # layer at a time into two alternating full-size buffers; their gradients pass through per-layer
    # staging slots (one slot per rank of the storage group, a shard each).
    storage = math.prod(mesh.get(a, 1) for a in ("fsdp", "data", "expert", "seq") if a != "data") or 1
    gather = staging = 0.0
    if storage > 1:
        for path, s in specs:
            if "/repeat/" in path and len(s.shape) >= 3 and _shard_fraction(s, mesh) < 1.0:
                per_layer = math.prod(s.shape[1:])
                tp = mesh.get("model", 1) if any("model" in _axis_names(e) for e in (s.mesh_axes or ())) else 1
                gather += 2 * 2.0 * per_layer / tp
                staging += 2.0 * math.prod(s.shape) * _shard_fraction(s, mesh) * storage
    if gather:
        out["FSDP gather buffers (2 layers)"] = gather
        out["gradient reduce-scatter staging"] = staging
    # Activations.
    dec = trainer_cfg.model.decoder
    d = dec.dim
    layers = dec.transformer.num_layers
    batch_axes = math.prod(mesh.get(a, 1) for a in ("data", "expert", "fsdp"))
    if per_gpu_batch is None:
        global_batch = getattr(trainer_cfg.input, "global_batch_size", None) or batch_axes
        per_gpu_batch = max(1, global_batch // batch_axes)
    seq_len = seq_len or getattr(trainer_cfg.input, "source_length", None) or 4096
    seq_local = seq_len // mesh.get("seq", 1)
    tokens = per_gpu_batch * seq_local
    out["layer-input checkpoints (full remat)"] = float(act_bytes) * tokens * d * layers
    ffn = getattr(dec.transformer.layer.feed_forward, "hidden_dim", None)
    ffn = ffn if isinstance(ffn, int) else int(8 / 3 * d)
    tp = mesh.get("model", 1)
    # One layer's live set while it is recomputed and differentiated: qkv, attention output, two
    # FFN projections, their product, and as much again for gradients.
    out["one layer's working set"] = float(act_bytes) * tokens * (4 * d + 3 * ffn // tp) * 2
    chunk = getattr(trainer_cfg.model, "scan_chunk", None) or tokens
    out["logits chunk of the fused loss (fp32 + bf16)"] = 6.0 * min(chunk, tokens) * dec.vocab_size / tp
    return MemoryPlan(num_gpus=num_gpus, mesh=mesh, total_params=total, local_params=local, bytes_per_gpu=out,
                      hbm_bytes=hbm_gb * 1e9)


@dataclasses.dataclass
class CostAnalysis:
    """What a training step costs per GPU, from the config alone (the counterpart of the compiled
    executable's cost analysis the reference prints without hardware,
    axlearn/common/aot_compilation.py): matrix FLOPs, attention FLOPs, bytes the optimizer streams,
    bytes every collective moves, and a step-time estimate from given peak rates."""

    tokens_per_gpu: int
    gemm_flops: float            # projections + LM head, forward + backward (+ recomputed forward)
    attention_flops: float       # causal QK^T / PV, forward + backward (+ recomputed forward)
    optimizer_bytes: float       # fp32 master + moments read and written, gradient read, bf16 copy written
    collective_bytes: dict       # name -> bytes received per GPU and step
    gemm_tflops: float
    attention_tflops: float
    hbm_gbs: float
    link_gbs: float

    @property
    def compute_ms(self) -> float:
        return 1e3 * (self.gemm_flops / (self.gemm_tflops * 1e12) + self.attention_flops / (self.attention_tflops * 1e12)
                      + self.optimizer_bytes / (self.hbm_gbs * 1e9))

    @property
    def collective_ms(self) -> float:
        return 1e3 * sum(self.collective_bytes.values()) / (self.link_gbs * 1e9)

    def table(self) -> str:
        lines = [f"per GPU and step: {self.tokens_per_gpu} tokens",
                 f"  GEMM work                   {self.gemm_flops / 1e12:10.1f} TFLOP  ({self.gemm_tflops:.0f} TFLOP/s assumed)",
                 f"  attention work              {self.attention_flops / 1e12:10.1f} TFLOP  ({self.attention_tflops:.0f} TFLOP/s assumed)",
                 f"  optimizer traffic           {self.optimizer_bytes / 1e9:10.1f} GB     ({self.hbm_gbs:.0f} GB/s assumed)"]
        for name, b in self.collective_bytes.items():
            lines.append(f"  {name:<27} {b / 1e9:10.2f} GB received over NVLink ({self.link_gbs:.0f} GB/s assumed)")
        lines.append(f"  compute estimate            {self.compute_ms:10.1f} ms; collectives {self.collective_ms:.1f} ms "
                     f"(hidden when they overlap the GEMMs)")
        lines.append(f"  tokens/s per GPU at the compute estimate: {self.tokens_per_gpu / self.compute_ms * 1e3:,.0f}")
        return "\n".join(lines)


def analyze_training_cost(trainer_cfg, *, num_gpus: int, per_gpu_batch: Optional[int] = None,
                          seq_len: Optional[int] = None, full_remat: bool = True, gemm_tflops: float = 1377.0,
                          attention_tflops: float = 800.0, hbm_gbs: float = 6551.0, link_gbs: float = 770.0,
                          moment_count: int = 2) -> CostAnalysis:
    """Defaults: the sustained library GEMM rate, copy bandwidth and peer-copy bandwidth measured on
    B200, and this framework's attention kernels' rate."""
    names = tuple(trainer_cfg.mesh_axis_names)
    shape = infer_mesh_shape(tuple(trainer_cfg.mesh_shape), num_devices=num_gpus)
    mesh = dict(zip(names, shape))
    model = trainer_cfg.model.clone(name="model").instantiate(parent=None)
    specs = flatten_items(model.create_parameter_specs_recursively(), is_leaf=lambda x: hasattr(x, "mesh_axes"))
    dec = trainer_cfg.model.decoder
    d, layers = dec.dim, dec.transformer.num_layers
    tp, sp = mesh.get("model", 1), mesh.get("seq", 1)
    batch_axes = math.prod(mesh.get(a, 1) for a in ("data", "expert", "fsdp"))
    if per_gpu_batch is None:
        global_batch = getattr(trainer_cfg.input, "global_batch_size", None) or batch_axes
        per_gpu_batch = max(1, global_batch // batch_axes)
    seq_len = seq_len or getattr(trainer_cfg.input, "source_length", None) or 4096
    tokens = per_gpu_batch * seq_len // sp
    # Every matrix parameter (>= 2 dims, embeddings excluded: a lookup, not a product) costs
    # 2 FLOPs per element and token forward and 4 backward; full remat repeats the forward of the
    # layer stack.
    # (Stacked parameters carry a leading layer dim: a stacked norm scale is [L, D], not a matrix.)
    matrix_stack = sum(math.prod(sp_.shape) for path, sp_ in specs if len(sp_.shape) >= 3 and "/repeat/" in path)
    matrix_rest = sum(math.prod(sp_.shape) for path, sp_ in specs
                      if len(sp_.shape) >= 2 and "/repeat/" not in path and "emb" not in path.split("/")[-2:][0])
    shared_head = not any("lm_head" in path for path, _ in specs)
    if shared_head:
        matrix_rest += dec.vocab_size * d        # the embedding doubles as the output projection
    passes_stack = 8.0 if full_remat else 6.0
    gemm = tokens * (passes_stack * matrix_stack + 6.0 * matrix_rest) / tp
    # Causal attention: 4 * T * T * d / 2 FLOPs per sequence forward, 2.5x that backward.
    per_seq = 4.0 * seq_len * seq_len * d * 0.5
    attention = per_gpu_batch * layers * per_seq * ((2.0 if full_remat else 1.0) + 2.5) / (tp * sp)
    local = sum(math.prod(s_.shape) * _shard_fraction(s_, mesh) for _, s_ in specs)
    optimizer = local * (4.0 * 2 * (1 + moment_count) + 2.0 + 2.0)
    coll: dict = {}
    storage = math.prod(mesh.get(a, 1) for a in ("fsdp", "expert", "seq")) or 1
    if storage > 1:
        sharded = sum(math.prod(s_.shape) for _, s_ in specs if _shard_fraction(s_, mesh) < 1.0) / tp
        frac = (storage - 1) / storage
        coll["parameter all-gathers"] = 2.0 * sharded * frac * (3.0 if full_remat else 2.0)
        coll["gradient reduce-scatters"] = 2.0 * sharded * frac
    if tp > 1:
        # Two all-reduces forward (attention output, FFN output) and two backward per layer pass.
        per_layer = 2.0 * tokens * d * 2.0 * (tp - 1) / tp
        coll["tensor-parallel all-reduces"] = per_layer * layers * ((2.0 if full_remat else 1.0) + 1.0) * 2.0
    if mesh.get("data", 1) > 1:
        coll["data-parallel gradient all-reduce"] = 2.0 * 2.0 * local * (mesh["data"] - 1) / mesh["data"]
    return CostAnalysis(tokens_per_gpu=tokens, gemm_flops=gemm, attention_flops=attention, optimizer_bytes=optimizer,
                        collective_bytes=coll, gemm_tflops=gemm_tflops, attention_tflops=attention_tflops,
                        hbm_gbs=hbm_gbs, link_gbs=link_gbs)


def main(argv: Optional[Sequence[str]] = None) -> int:
    from axlearn_b200.common.launch_trainer import _import

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--module", required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--num_gpus", type=int, default=None)
    ap.add_argument("--topology", default=None,
                    help="instead of --num_gpus / --hbm_gb: an instance type such as gpu-b200-64 or b200-8")
    ap.add_argument("--hbm_gb", type=float, default=None)
    ap.add_argument("--per_gpu_batch", type=int, default=None)
    ap.add_argument("--seq_len", type=int, default=None)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--cost", action="store_true", help="also print FLOPs, collective bytes and a step-time estimate")
    args = ap.parse_args(argv)
    if args.topology:
        from axlearn_b200.cloud.gcp.system_characteristics import parse_gpu_instance_type

        vm, num_vms = parse_gpu_instance_type(args.topology)
        args.num_gpus = args.num_gpus or vm.chips_per_vm * num_vms
        args.hbm_gb = args.hbm_gb or float(vm.memory_gb_per_chip)
    if not args.num_gpus:
        ap.error("one of --num_gpus or --topology is required")
    args.hbm_gb = args.hbm_gb or 180.0
    cfg = _import(args.module).named_trainer_configs()[args.config]()
    plan = plan_training_memory(cfg, num_gpus=args.num_gpus, hbm_gb=args.hbm_gb, per_gpu_batch=args.per_gpu_batch,
                                seq_len=args.seq_len)
    cost = analyze_training_cost(cfg, num_gpus=args.num_gpus, per_gpu_batch=args.per_gpu_batch,
                                 seq_len=args.seq_len) if args.cost else None
    if args.json:
        out = {"mesh": plan.mesh, "bytes_per_gpu": plan.bytes_per_gpu, "total_bytes": plan.total_bytes,
               "fits": plan.fits}
        if cost is not None:
            out["cost"] = {"gemm_flops": cost.gemm_flops, "attention_flops": cost.attention_flops,
                           "optimizer_bytes": cost.optimizer_bytes, "collective_bytes": cost.collective_bytes,
                           "compute_ms": cost.compute_ms, "collective_ms": cost.collective_ms}
        print(json.dumps(out))
    else:
        print(plan.table())
        if cost is not None:
            print(cost.table())
    return 0 if plan.fits else 1


if __name__ == "__main__":
    raise SystemExit(main())
