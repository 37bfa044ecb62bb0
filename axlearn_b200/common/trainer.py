"""SpmdTrainer: the training loop.

Parity targets in the reference (axlearn/common/trainer.py): ``SpmdTrainer.Config``
(:92-253), construction inside the mesh (:255-390), trainer-state partition specs (:355-373),
watchdog (:436-526), ``run`` (:580-697), ``init`` (:699-844), ``_prepare_training``
(:899-950), ``restore_checkpoint`` (:952-1023), ``save_checkpoint`` (:1025-1034),
``_run_step`` (:1136-1216), ``_train_step`` (:1281-1355), tracing (:1357-1411),
``select_mesh_config`` (:1414-1436).

Execution model: one process per GPU, eager dispatch.  A step is

    host batch (pinned) --H2D--> model forward on low-precision shadows --> backward
    (per-layer remat; FSDP gathers/scatters overlap on a side stream) --> gradient sync for
    replicated tensors --> ONE fused clip+AdamW kernel that updates fp32 masters, moments and
    the shadows --> summaries.

``TrainerState`` is ``{"prng_key": uint32[4], "model": <params>, "learner": <learner
state>}`` — the tree the checkpointer flattens into tensor names.
"""

from __future__ import annotations

import collections
import contextlib
import json
import math
import os
import signal
import threading
import time
from typing import Any, Optional, Sequence, Union

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import ParameterSpec, use_device
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.checkpointer import (
    EXACT,
    BaseCheckpointer,
    Checkpointer,
    CheckpointValidationType,
)
from axlearn_b200.common.config import (
    REQUIRED,
    ConfigModifier,
    InstantiableConfig,
    Required,
    config_class,
    maybe_instantiate,
)
from axlearn_b200.common.input_base import Input
from axlearn_b200.common.learner import Learner
from axlearn_b200.common.metrics import MetricAccumulator
from axlearn_b200.common.module import Module, OutputCollection, functional
from axlearn_b200.common.optimizer_base import OptParam
from axlearn_b200.common.summary_writer import BaseWriter, SummaryWriter
from axlearn_b200.common.utils import (
    TensorSpec,
    VDict,
    count_model_params,
    flatten_items,
    thread_stack_traces,
    tree_map,
)
from axlearn_b200.parallel import collectives as coll
from axlearn_b200.parallel import fsdp, grad_sync
from axlearn_b200.parallel.mesh import (
    HybridMeshShape,
    Mesh,
    MeshShape,
    create_mesh,
    infer_mesh_shape,
    select_mesh_rule,
)

Tensor = torch.Tensor
_is_spec = lambda x: isinstance(x, TensorSpec)


class UndefinedLossException(RuntimeError):
    """The training loss became NaN or infinite."""


def select_mesh_config(trainer_config: "SpmdTrainer.Config", *, mesh_selector: str) -> None:
    """Applies the first mesh rule whose regex fully matches ``mesh_selector``: a mesh shape
    replaces ``mesh_shape``; a ConfigModifier config rewrites the whole trainer config."""
    matched, rule = select_mesh_rule(mesh_selector, trainer_config.mesh_rules)
    if not matched or rule is None:
        return
    if isinstance(rule, InstantiableConfig):
        modifier = rule.instantiate()
        new = modifier(trainer_config)
        for k, v in new.items():
            if k != "klass":
                setattr(trainer_config, k, v)
    else:
        trainer_config.mesh_shape = rule


class SpmdTrainer(Module):
    @config_class
    class Config(Module.Config):
        input: Required[InstantiableConfig] = REQUIRED
        model: Required[InstantiableConfig] = REQUIRED
        learner: Required[InstantiableConfig] = REQUIRED
        # Root directory: checkpoints/ and summaries/ are created below it.
        dir: Required[str] = REQUIRED
        # Mesh: one entry per name in mesh_axis_names; a single -1 is inferred.
        mesh_shape: Required[Union[MeshShape, HybridMeshShape]] = REQUIRED
        mesh_axis_names: Required[Sequence[str]] = REQUIRED
        # Ordered (regex, mesh shape | ConfigModifier config) chosen by --mesh_selector.
        mesh_rules: Optional[Sequence[tuple[str, Any]]] = None
        batch_axis_names: Union[str, Sequence[str]] = "data"
        checkpointer: InstantiableConfig = Checkpointer.default_config()
        init_state_builder: Optional[InstantiableConfig] = None
        summary_writer: InstantiableConfig = SummaryWriter.default_config()
        evalers: dict[str, InstantiableConfig] = {}
        max_step: Optional[int] = None
        # dtype of the forward/backward pass; None = parameter dtype.
        train_dtype: Optional[torch.dtype] = None
        log_every_n_steps: int = 100
        # Profiler traces.
        start_trace_steps: Sequence[int] = []
        start_trace_process_indices: Union[str, Sequence[int]] = [0]
        n_steps_for_each_trace: int = 3
        # Hang detection.
        watchdog_timeout_seconds: Optional[float] = None
        crash_on_hang_timeout_seconds: Optional[float] = None
        device_monitor: Optional[InstantiableConfig] = None
        recorder: Optional[InstantiableConfig] = None
        save_input_iterator: bool = False
        # Micro-batches per optimizer step (the per-process batch is split along dim 0 and the
        # gradients are averaged); see GradientAccumulationModifier.
        grad_accumulation_steps: int = 1
        prune_empty_state_updates: bool = True
        # Device to train on; None = cuda:LOCAL_RANK when available else cpu.
        device: Optional[str] = None

    def __init__(self, cfg: "SpmdTrainer.Config", *, parent: Optional[Module] = None, mesh: Optional[Mesh] = None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True
        if cfg.model.dtype is None:
            raise ValueError("cfg.model.dtype must be set (the dtype parameters are stored in)")
        self._step = 0
        self._trainer_state: Optional[dict] = None
        self._shadows: Optional[Any] = None
        self._has_param_noise = False
        self._device = torch.device(cfg.device) if cfg.device else _default_device()
        self._mesh = mesh or create_mesh(cfg.mesh_shape, cfg.mesh_axis_names)
        self._step_times = collections.deque(maxlen=100)
        self._watchdog_stop = threading.Event()
        self._watchdog_thread: Optional[threading.Thread] = None
        self._profiler = None
        self._trace_stop_step: Optional[int] = None
        with self._mesh, use_device(self._device):
            self._add_child("input", cfg.input.clone())
            self._add_child(
                "summary_writer",
                cfg.summary_writer.clone(dir=cfg.summary_writer.dir or os.path.join(cfg.dir, "summaries", "train_train")),
            )
            self._add_child("model", cfg.model)
            self._has_param_noise = bool(getattr(self.model, "has_parameter_noise", lambda: False)())
            self._add_child("learner", cfg.learner)
            self._add_child(
                "checkpointer",
                cfg.checkpointer.clone(dir=getattr(cfg.checkpointer, "dir", None) or os.path.join(cfg.dir, "checkpoints")),
            )
            if cfg.init_state_builder is not None:
                self._add_child("init_state_builder", cfg.init_state_builder)
            self._evalers = {}
            for name, ecfg in cfg.evalers.items():
                ecfg = ecfg.clone()
                if "summary_writer" in ecfg and ecfg.summary_writer is not None and not ecfg.summary_writer.dir:
                    ecfg.summary_writer.dir = os.path.join(cfg.dir, "summaries", name)
                self._evalers[name] = self._add_child(name, ecfg, model=self.model) if _takes_model(ecfg) else self._add_child(name, ecfg)
            self._model_param_specs = self.model.create_parameter_specs_recursively()
            self._learner_state_specs = self.learner.create_state_partition_specs(self._model_param_specs)
        if cfg.device_monitor is not None:
            self._device_monitor = cfg.device_monitor.instantiate()
        else:
            self._device_monitor = None
        self._recorder = maybe_instantiate(cfg.recorder)

    # ------------------------------------------------------------------ properties
    @property
    def step(self) -> int:
        return self._step

    @property
    def trainer_state(self) -> dict:
        return self._trainer_state

    @property
    def mesh_obj(self) -> Mesh:
        return self._mesh

    def mesh(self) -> Mesh:
        return self._mesh

    @property
    def trainer_state_specs(self) -> dict:
        return {
            "prng_key": TensorSpec(shape=(4,), dtype=torch.uint32, mesh_axes=(None,)),
            "model": self._model_param_specs,
            "learner": self._learner_state_specs,
        }

    def model_params_for_eval(self) -> Any:
        state = self._trainer_state
        if "ema" in state["learner"]:
            return state["learner"]["ema"].ema
        return self._shadows if self._shadows is not None else state["model"]

    # ------------------------------------------------------------------ init / restore
    def init(self, prng_key: Tensor) -> None:
        """Fresh state: parameters (optionally completed from ``init_state_builder``),
        learner state, shadows."""
        cfg = self._config
        with self._mesh, use_device(self._device):
            param_key, self_key = prng.split(prng_key, 2)
            prebuilt = None
            if "init_state_builder" in self._children:
                prebuilt = self.init_state_builder.prebuilt_model_params(self)
            model_params = self.model.initialize_parameters_recursively(param_key, prebuilt=prebuilt, device=self._device)
            model_params = tree_map(lambda t: t.to(self._device), model_params)
            learner_state = self.learner.init(self._opt_params(model_params))
            learner_state = _to_device(learner_state, self._device)
            self._trainer_state = {"prng_key": self_key, "model": model_params, "learner": learner_state}
            self._build_shadows()

    def _opt_params(self, model_params: Any) -> Any:
        specs = dict(flatten_items(self._model_param_specs, is_leaf=_is_spec))
        from axlearn_b200.common.utils import unflatten_items

        return unflatten_items([
            (p, OptParam(t, getattr(specs.get(p), "factorization", None), getattr(specs.get(p), "weight_decay_scale", None)))
            for p, t in flatten_items(model_params)
        ])

    def _build_shadows(self) -> None:
        """Low-precision copies of float parameters that the forward pass reads (identical to
        the masters when train_dtype is the parameter dtype)."""
        cfg = self._config
        types = dict(flatten_items(self.learner.update_types(self._model_param_specs)))
        from axlearn_b200.common.learner import should_update_with_optimizers, UpdateType

        def mk(path: str, t: Tensor) -> Tensor:
            trainable = t.is_floating_point() and should_update_with_optimizers(types.get(path, UpdateType.ALL_UPDATES))
            if cfg.train_dtype is not None and t.is_floating_point() and t.dtype != cfg.train_dtype:
                s = t.detach().to(cfg.train_dtype)
            else:
                s = t.detach()
            return s.requires_grad_(trainable)

        from axlearn_b200.common.utils import tree_paths

        self._shadows = tree_map(lambda t, p: mk(p, t), self._trainer_state["model"], tree_paths(self._trainer_state["model"]))
        self._place_sharded_shadows_in_symmetric_memory()

    def _place_sharded_shadows_in_symmetric_memory(self) -> None:
        """Storage-sharded stacked shadows are moved into peer-mapped memory so that the fused
        FSDP kernels of the other ranks can read this rank's shards over NVLink."""
        from axlearn_b200.parallel import fsdp_fused

        mesh = self._mesh
        if self._device.type != "cuda" or mesh.size == 1 or not mesh._real or not fsdp_fused.ENABLED:  # pylint: disable=protected-access
            return
        specs = dict(flatten_items(self._model_param_specs, is_leaf=_is_spec))

        def visit(node, prefix, stacked):
            if isinstance(node, dict):
                for k in list(node.keys()):
                    path = f"{prefix}/{k}" if prefix else str(k)
                    v = node[k]
                    if isinstance(v, Tensor):
                        spec = specs.get(path)
                        if not (stacked or isinstance(node, VDict)) or spec is None or spec.mesh_axes is None:
                            continue
                        if v.dtype != torch.bfloat16 or not v.requires_grad:
                            continue
                        plan = fsdp.LeafPlan(mesh, tuple(spec.mesh_axes)[1:])
                        if plan.world > 1 and plan.world <= 8:
                            node[k] = fsdp_fused.make_symmetric(v.detach(), plan).requires_grad_(True)
                    else:
                        visit(v, path, stacked or isinstance(node, VDict))

        visit(self._shadows, "", False)

    def restore_checkpoint(self, restore_step: Optional[int] = None) -> Optional[int]:
        """Restores the latest (or given) checkpoint into this trainer; returns its step or
        None when there is none."""
        cfg = self._config
        with self._mesh, use_device(self._device):
            target = self._state_structure()
            if cfg.save_input_iterator:
                target["input_iter"] = self.input
            try:
                step, restored = self.checkpointer.restore(
                    step=restore_step, state=target, specs=self.trainer_state_specs, device=self._device)
            except ValueError:
                if not cfg.save_input_iterator:
                    raise
                target.pop("input_iter")
                step, restored = self.checkpointer.restore(
                    step=restore_step, state=target, specs=self.trainer_state_specs, device=self._device)
            if step is None:
                return None
            restored.pop("input_iter", None)
            restored["prng_key"] = restored["prng_key"].cpu()
            restored["learner"] = _host_scalars(restored["learner"])
            self._trainer_state = restored
            self._step = step
            self._build_shadows()
            return step

    def _state_structure(self) -> dict:
        """Target structure for restore: TensorSpecs with *local* (shard) shapes."""
        mesh = self._mesh

        def localise(spec):
            shape = mesh.shard_shape(spec.shape, spec.mesh_axes) if spec.mesh_axes is not None and spec.shape is not None and len(spec.mesh_axes) == len(spec.shape) else tuple(spec.shape)
            return TensorSpec(shape=shape, dtype=spec.dtype, mesh_axes=spec.mesh_axes)

        if self._trainer_state is not None:
            return {k: v for k, v in self._trainer_state.items()}
        specs = self.trainer_state_specs
        return tree_map(localise, specs, is_leaf=_is_spec)

    def _check_device_status(self) -> None:
        """Raises ``RuntimeError`` when a kernel reported a bounded-wait time-out since the last
        check (its outputs may be partly unwritten, so the step must not be kept)."""
        if self._device.type != "cuda":
            return
        from axlearn_b200.ops import cuda_ops

        cuda_ops.check_status(self._device)

    def save_checkpoint(self, evaler_summaries: Optional[dict] = None, *, force: bool = False) -> bool:
        cfg = self._config
        with self._mesh:
            state = dict(self._trainer_state)
            if cfg.save_input_iterator:
                state["input_iter"] = self.input
            # Never persist a state that a timed-out kernel may have corrupted: the check raises,
            # the error propagates and the supervising agent restarts from the last good checkpoint.
            saved = self.checkpointer.save(
                step=self._step, state=state, specs=self.trainer_state_specs,
                evaler_summaries=evaler_summaries, force=force, pre_save_check=self._check_device_status)
        return saved

    # ------------------------------------------------------------------ run
    def run(self, prng_key: Tensor, *, return_evaler_summaries: bool = False) -> Optional[dict]:
        """Trains until ``max_step`` (or input exhaustion); returns the last step's outputs."""
        cfg = self._config
        output = None
        from axlearn_b200.common import measurement

        def record(event, *args):
            if self._recorder is not None:
                self._recorder.record(event, *args)

        record(measurement.Event.START_JOB)
        if self._recorder is not None:
            self._recorder.start_monitoring()
        try:
            with self._watchdog(), self._mesh, use_device(self._device), self.checkpointer:
                if self._device_monitor is not None:
                    self._device_monitor.start_monitoring()
                record(measurement.Event.START_TRAINING_PREPARATION)
                self._prepare_training(prng_key)
                record(measurement.Event.END_TRAINING_PREPARATION)
                input_iter = self.input.batches(iter(self.input.dataset()))
                while True:
                    if cfg.max_step is not None and self._step >= cfg.max_step:
                        break
                    record(measurement.Event.START_DATA_LOADING)
                    batch = next(input_iter, None)
                    record(measurement.Event.END_DATA_LOADING)
                    if batch is None:
                        break
                    self._maybe_trace()
                    self._step += 1
                    record(measurement.Event.START_STEP, self._step)
                    t0 = time.perf_counter()
                    output = self._run_step(batch)
                    self._step_times.append(time.perf_counter() - t0)
                self._stop_trace()
                self.checkpointer.wait_until_finished()
                self.summary_writer.flush()
                if self._device_monitor is not None:
                    self._device_monitor.stop_monitoring()
        finally:
            record(measurement.Event.END_JOB)
        return output

    def _prepare_training(self, prng_key: Tensor) -> None:
        cfg = self._config
        os.makedirs(cfg.dir, exist_ok=True)
        restored = self.restore_checkpoint()
        if restored is None:
            self.init(prng_key)
            self._step = 0
            self.save_checkpoint(self._run_eval())
        self._log_state()
        self.summary_writer.log_config(cfg, step=self._step)

    def _log_state(self) -> None:
        cfg = self._config
        if coll.process_index() != 0:
            return
        lines = [f"{p}: {tuple(t.shape)} {t.dtype}" for p, t in flatten_items(self._trainer_state) if isinstance(t, Tensor)]
        with open(os.path.join(cfg.dir, "trainer_state_tree.txt"), "w") as f:
            f.write("\n".join(lines))
        with open(os.path.join(cfg.dir, "model_analysis.txt"), "w") as f:
            f.write(self.model_analysis())

    def model_analysis(self) -> str:
        specs = flatten_items(self._model_param_specs, is_leaf=_is_spec)
        total = sum(math.prod(s.shape) for _, s in specs)
        lines = [f"{p:<100} {str(tuple(s.shape)):<28} {s.mesh_axes}" for p, s in specs]
        local = count_model_params(self._trainer_state["model"]) if self._trainer_state else 0
        lines.append(f"Total model params: {total:,}; local shard params: {local:,}")
        return "\n".join(lines)

    # ------------------------------------------------------------------ step
    def train_step(self, host_batch: dict) -> dict:
        """One optimisation step on a per-process host batch: asynchronous host→device copy of
        the inputs, forward, backward, update.  Returns ``{"loss", "aux", "summaries"}`` with
        ``loss`` still on the device (reading it is the caller's device→host sync).  The
        trainer must have been initialised (``init`` or ``restore_checkpoint``)."""
        with self._mesh, use_device(self._device):
            batch = tree_map(
                lambda t: t.to(self._device, non_blocking=True) if isinstance(t, Tensor) else t, host_batch)
            self._step += 1
            return self._train_step(batch)

    def _run_step(self, host_batch: dict) -> dict:
        cfg = self._config
        batch = tree_map(lambda t: t.to(self._device, non_blocking=True) if isinstance(t, Tensor) else t, host_batch)
        out = self._train_step(batch)
        step = self._step
        if step <= 5 or step % cfg.log_every_n_steps == 0:
            loss = float(out["loss"])
            # The loss read above synchronised the device: a bounded wait that gave up inside a
            # kernel (late peer, lost flag) has left its code in the status word by now.
            self._check_device_status()
            if not math.isfinite(loss):
                raise UndefinedLossException(f"loss is {loss} at step {step}")
            if coll.process_index() == 0:
                avg = sum(self._step_times) / max(1, len(self._step_times))
                print(f"[trainer] step {step} loss {loss:.6f} avg_step_s {avg:.4f}", flush=True)
        self.summary_writer(step, {"loss": out["loss"], **out["summaries"]})
        evaler_summaries = self._run_eval()
        self.save_checkpoint(evaler_summaries)
        return out

    def _train_step(self, batch: dict) -> dict:
        """Forward, backward and update on one per-process batch (already on device)."""
        cfg = self._config
        state = self._trainer_state
        new_key, _noise_key, fwd_key, _learner_key = prng.split(state["prng_key"], 4)
        batch = _shard_sequence(self.input.dispatch_global_batch(batch), self._mesh)
        self._zero_grads()
        steps = max(1, cfg.grad_accumulation_steps)
        micro_batches = _split_batch(batch, steps)
        fwd_keys = prng.split(fwd_key, steps) if steps > 1 else [fwd_key]
        loss, aux, oc = None, None, None
        acc = MetricAccumulator() if steps > 1 else None
        pipeline_scale = 1.0 / self._mesh.shape.get("pipeline", 1) if self._mesh is not None else 1.0
        for micro, key in zip(micro_batches, fwd_keys):
            if self._device.type == "cuda":
                from axlearn_b200.parallel import fsdp_fused

                # Cross-rank ordering of the gradient staging buffers (once per micro-batch).
                fsdp_fused.begin_step_all(accumulate=micro is not micro_batches[0])
            # Parameter noise (if any layer configures it) perturbs what the model reads; gradients
            # still land on the clean shadows (reference: axlearn/common/trainer.py:1305-1307).
            step_params = self._shadows
            if self._has_param_noise:
                step_params = self.model.apply_parameter_noise_recursively(_noise_key, self._shadows)
            (micro_loss, aux), oc = functional(
                self.model, key, step_params, [micro], is_training=True, method="forward")
            # Micro-batch gradients are averaged (reference: gradient_accumulation.py:96-351).
            # Pipeline ranks each hold 1/num_stages of the loss gradient (see common/pipeline.py).
            (micro_loss * (pipeline_scale / steps)).backward()
            loss = micro_loss.detach() / steps if loss is None else loss + micro_loss.detach() / steps
            if acc is not None:
                acc.update(oc.summaries)
        if acc is not None:
            oc.summaries.clear()
            oc.summaries.update(acc.summaries())
        fsdp.wait_pending(self._device if self._device.type == "cuda" else None)
        if self._mesh is not None and self._mesh.shape.get("pipeline", 1) > 1:
            # A stage that does not touch a replicated parameter still takes part in its reduction.
            for _, sh in flatten_items(self._shadows):
                if isinstance(sh, Tensor) and sh.requires_grad and sh.grad is None:
                    sh.grad = torch.zeros_like(sh)
        grads = tree_map(lambda s: s.grad if s.requires_grad else None, self._shadows)
        grad_sync.sync_grads(grads, specs=self._model_param_specs, mesh=self._mesh)
        summaries = {"model": oc.summaries}
        learner_oc = OutputCollection({}, {}, {})
        from axlearn_b200.common.module import InvocationContext, set_current_context

        lctx = InvocationContext(name="learner", parent=None, module=self.learner, state=None,
                                 is_training=True, prng_key=None, output_collection=learner_oc)
        with set_current_context(lctx, require_parent=False):
            state["learner"] = self.learner.update(
                model_params=state["model"], gradients=grads, state=state["learner"],
                param_specs=self._model_param_specs, state_updates=oc.state_updates, shadows=self._shadows)
        summaries["learner"] = learner_oc.summaries
        if self._device.type == "cuda":
            fsdp_fused.invalidate_all()  # the shards changed: gather buffers are stale
        state["prng_key"] = new_key
        # Each rank's loss is its share of the global mean (normalised by the global number of
        # live targets); the reported loss is the sum of the shares over the batch axes.
        global_loss = coll.all_reduce_scalar(loss.detach().float(), ("data", "expert", "fsdp", "seq"))
        return {"loss": global_loss, "aux": aux, "summaries": summaries}

    def _zero_grads(self) -> None:
        def visit(node, stacked):
            if isinstance(node, Tensor):
                if stacked and node.requires_grad:
                    # Stacked leaves keep one persistent gradient buffer that the layer loop
                    # fills slice by slice.
                    if node.grad is None:
                        node.grad = torch.empty_like(node)
                    fsdp.reset_grad_slices(node)
                else:
                    node.grad = None
            elif isinstance(node, dict):
                for v in node.values():
                    visit(v, stacked or isinstance(node, VDict))

        visit(self._shadows, False)

    def _run_eval(self) -> dict:
        out = {}
        for name, evaler in self._evalers.items():
            _, summaries, _ = evaler.eval_step(
                self._step, prng_key=self._trainer_state["prng_key"], model_params=self.model_params_for_eval())
            out[name] = summaries
        return out

    # ------------------------------------------------------------------ tracing
    def _maybe_trace(self) -> None:
        cfg = self._config
        if self._trace_stop_step is not None and self._step >= self._trace_stop_step:
            self._stop_trace()
        if self._step in cfg.start_trace_steps and self._should_trace_here():
            out_dir = os.path.join(cfg.dir, "summaries", "train_train", f"trace_step{self._step}")
            os.makedirs(out_dir, exist_ok=True)
            acts = [torch.profiler.ProfilerActivity.CPU]
            if self._device.type == "cuda":
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._profiler = torch.profiler.profile(activities=acts)
            self._profiler.__enter__()
            self._trace_dir = out_dir
            self._trace_stop_step = self._step + cfg.n_steps_for_each_trace

    def _should_trace_here(self) -> bool:
        idx = self._config.start_trace_process_indices
        return idx == "all" or coll.process_index() in idx

    def _stop_trace(self) -> None:
        if self._profiler is not None:
            self._profiler.__exit__(None, None, None)
            try:
                self._profiler.export_chrome_trace(os.path.join(self._trace_dir, f"trace_{coll.process_index()}.json"))
            except Exception:  # pylint: disable=broad-except
                pass
            self._profiler = None
        self._trace_stop_step = None

    # ------------------------------------------------------------------ watchdog
    @contextlib.contextmanager
    def _watchdog(self):
        cfg = self._config
        if not cfg.watchdog_timeout_seconds:
            yield
            return
        self._watchdog_stop.clear()
        self._watchdog_thread = threading.Thread(target=self._watchdog_loop, name="trainer-watchdog", daemon=True)
        self._watchdog_thread.start()
        try:
            yield
        finally:
            self._watchdog_stop.set()
            self._watchdog_thread.join(timeout=5)

    def _watchdog_loop(self) -> None:
        cfg = self._config
        last_step, last_change = self._step, time.time()
        poll = min(1.0, cfg.watchdog_timeout_seconds / 4)
        while not self._watchdog_stop.wait(poll):
            if self._step != last_step:
                last_step, last_change = self._step, time.time()
                continue
            stalled = time.time() - last_change
            if stalled >= cfg.watchdog_timeout_seconds:
                idle = self._device_monitor.is_host_idle() if self._device_monitor is not None else None
                self.watchdog_report = "\n".join("\n".join(t) for t in thread_stack_traces())
                print(f"[watchdog] step {last_step} unchanged for {stalled:.1f}s (host idle: {idle})\n"
                      f"{self.watchdog_report}", flush=True)
                if cfg.crash_on_hang_timeout_seconds and stalled >= cfg.crash_on_hang_timeout_seconds and self._trainer_state is not None:
                    os.kill(os.getpid(), signal.SIGKILL)
                last_change = time.time() if not cfg.crash_on_hang_timeout_seconds else last_change


def _shard_sequence(batch: dict, mesh) -> dict:
    """Sequence parallelism (``seq`` mesh axis): every rank of a ``seq`` group receives the same
    rows and keeps its contiguous slice of the time dim of each ``[B, T, ...]`` tensor."""
    if mesh is None or "seq" not in mesh.shape or mesh.shape["seq"] == 1:
        return batch
    s, r = mesh.shape["seq"], mesh.coords["seq"]

    def cut(t):
        if not isinstance(t, Tensor) or t.dim() < 2:
            return t
        if t.shape[1] % s:
            raise ValueError(f"sequence length {t.shape[1]} is not divisible by the seq axis ({s})")
        n = t.shape[1] // s
        return t[:, r * n:(r + 1) * n].contiguous()

    return tree_map(cut, batch)


def _split_batch(batch: dict, steps: int) -> list:
    """Splits every tensor of a batch into ``steps`` equal chunks along dim 0."""
    if steps == 1:
        return [batch]
    sizes = {t.shape[0] for _, t in flatten_items(batch) if isinstance(t, Tensor) and t.dim() > 0}
    if any(n % steps for n in sizes):
        raise ValueError(f"per-process batch sizes {sorted(sizes)} are not divisible by {steps} accumulation steps")
    return [tree_map(lambda t, i=i: t.chunk(steps, dim=0)[i] if isinstance(t, Tensor) and t.dim() > 0 else t, batch)
            for i in range(steps)]


def _takes_model(cfg) -> bool:
    import inspect

    klass = getattr(cfg, "klass", None)
    if klass is None:
        return False
    return "model" in inspect.signature(klass.__init__).parameters


def _default_device() -> torch.device:
    if torch.cuda.is_available():
        idx = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(idx)
        return torch.device("cuda", idx)
    return torch.device("cpu")


def _to_device(tree: Any, device: torch.device) -> Any:
    """Moves tensors with >= 1 dim to ``device``; 0-d counters stay on the host."""
    return tree_map(lambda t: t.to(device) if isinstance(t, Tensor) and t.dim() > 0 else t, tree)


def _host_scalars(tree: Any) -> Any:
    return tree_map(lambda t: t.cpu() if isinstance(t, Tensor) and t.dim() == 0 and t.dtype in (torch.int32, torch.int64) else t, tree)
