"""Evaluation during (or outside of) training.

Parity targets in the reference (axlearn/common/evaler.py): ``BaseMetricCalculator`` (:45),
``ModelSummaryAccumulator`` (:269) -- runs the model's forward on every eval batch and accumulates
the summaries it emits; ``CompositeMetricCalculator`` (:361) -- several calculators, optionally
fed by each other's outputs; ``EvalPolicy`` / ``every_n_steps_policy`` (:524-558);
``SpmdEvaler`` (:561-760) -- owns an eval input, a metric calculator and a summary writer, and
``eval_step(step, prng_key=, model_params=)`` returns ``(prng_key, summaries, outputs)``;
``GlobalMetricCalculator`` (:767) -- gathers per-example predictions for metrics that are not sums
over batches.

Eval runs under ``torch.no_grad`` with the trainer's (bf16) parameters; weighted summaries are
combined across ranks of the batch axes by their weights.
"""

from __future__ import annotations

import os
import time
from typing import Any, Callable, NamedTuple, Optional, Protocol, Sequence

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.config import (
    REQUIRED,
    InstantiableConfig,
    Required,
    config_class,
    config_for_function,
    maybe_set_config,
)
from axlearn_b200.common.metrics import MetricAccumulator, MetricSummary, WeightedSummary
from axlearn_b200.common.module import Module, functional
from axlearn_b200.common.summary_writer import SummaryWriter
from axlearn_b200.common.utils import flatten_items, tree_map

Tensor = torch.Tensor


class EvalPolicy(Protocol):
    def __call__(self, *, step: int, train_summaries: dict) -> bool: ...


def every_n_steps_policy(n: int = 1, *, min_step: int = 1, max_step: Optional[int] = None) -> EvalPolicy:
    """Evaluate at steps ``>= min_step`` that are multiples of ``n``, and at ``max_step``."""

    def fn(*, step: int, train_summaries: dict) -> bool:
        del train_summaries
        if step < min_step:
            return False
        return step % n == 0 or (max_step is not None and step == max_step)

    return fn


class BaseMetricCalculator(Module):
    """``init_state`` -> repeated ``forward(batch, model_params=, state=)`` -> ``get_summaries``."""

    @config_class
    class Config(Module.Config):
        eval_dtype: Optional[torch.dtype] = None
        prefix: Optional[str] = None

    def __init__(self, cfg, *, parent=None, model=None, model_param_partition_specs=None):
        super().__init__(cfg, parent=parent)
        self._model = model
        self._model_param_partition_specs = model_param_partition_specs
        self._allow_contextless = True

    def init_state(self, *, prng_key: Tensor, model_params: Any) -> Any:
        raise NotImplementedError(type(self))

    def forward(self, input_batch: dict, *, model_params: Any, state: Any) -> dict:
        """Returns ``{"state": ..., "output": ...}``."""
        raise NotImplementedError(type(self))

    def get_summaries(self, *, model_params: Any, state: Any, all_forward_outputs: list) -> dict:
        raise NotImplementedError(type(self))

    def _call_model(self, *, method: str, prng_key: Tensor, model_params: Any, input_batch: dict, **kwargs):
        cfg = self._config
        if cfg.eval_dtype is not None:
            input_batch = tree_map(
                lambda t: t.to(cfg.eval_dtype) if isinstance(t, Tensor) and t.is_floating_point() else t, input_batch)
        with torch.no_grad():
            return functional(self._model, prng_key, model_params, dict(input_batch=input_batch, **kwargs),
                              is_training=False, method=method)

    def formatted_metric_name(self, name: str) -> str:
        p = self._config.prefix
        return f"{p}/{name}" if p else name


class ModelSummaryAccumulator(BaseMetricCalculator):
    """Accumulates the summaries that ``model.<model_method>(input_batch)`` adds."""

    @config_class
    class Config(BaseMetricCalculator.Config):
        model_method: str = "forward"
        model_method_kwargs: dict = {}
        metric_accumulator: InstantiableConfig = MetricAccumulator.default_config()

    def __init__(self, cfg, *, parent=None, model=None, model_param_partition_specs=None):
        super().__init__(cfg, parent=parent, model=model, model_param_partition_specs=model_param_partition_specs)
        self._acc = cfg.metric_accumulator.instantiate()

    def init_state(self, *, prng_key, model_params):
        self._acc = self._config.metric_accumulator.instantiate()
        return {"prng_key": prng_key}

    def forward(self, input_batch, *, model_params, state):
        cfg = self._config
        key, next_key = prng.split(state["prng_key"], 2)
        outputs, oc = self._call_model(method=cfg.model_method, prng_key=key, model_params=model_params,
                                       input_batch=input_batch, **cfg.model_method_kwargs)
        self._acc.update(oc.summaries)
        return {"state": {"prng_key": next_key}, "output": self._per_example_outputs(outputs)}

    def _per_example_outputs(self, model_outputs):
        if isinstance(model_outputs, tuple) and len(model_outputs) == 2 and isinstance(model_outputs[1], dict):
            return {"loss": model_outputs[0], **model_outputs[1]}
        return model_outputs

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        return self._acc.summaries()


class CompositeMetricCalculator(BaseMetricCalculator):
    """Runs several calculators over the same batches; summaries are prefixed by their names.
    ``dependencies`` = ``(src, dst, dst_key)``: the output of ``src`` is added to the batch of
    ``dst`` under ``dst_key`` (so e.g. a metric can consume another calculator's predictions)."""

    @config_class
    class Config(BaseMetricCalculator.Config):
        metric_calculators: Required[dict] = REQUIRED
        dependencies: Sequence[tuple] = []

    def __init__(self, cfg, *, parent=None, model=None, model_param_partition_specs=None):
        super().__init__(cfg, parent=parent, model=model, model_param_partition_specs=model_param_partition_specs)
        self._calcs = {}
        for name, c in cfg.metric_calculators.items():
            self._calcs[name] = self._add_child(
                name, c.clone(eval_dtype=cfg.eval_dtype), model=model,
                model_param_partition_specs=model_param_partition_specs)
        order = list(self._calcs)
        for src, dst, _ in cfg.dependencies:
            if src not in self._calcs or dst not in self._calcs:
                raise ValueError(f"unknown calculator in dependency {src} -> {dst}")
            if order.index(src) > order.index(dst):
                raise ValueError(f"calculator {dst} depends on {src}, which runs later")

    def init_state(self, *, prng_key, model_params):
        keys = prng.split(prng_key, len(self._calcs))
        return {n: c.init_state(prng_key=k, model_params=model_params) for (n, c), k in zip(self._calcs.items(), keys)}

    def forward(self, input_batch, *, model_params, state):
        outputs, new_state = {}, {}
        for name, calc in self._calcs.items():
            batch = dict(input_batch)
            for src, dst, key in self._config.dependencies:
                if dst == name:
                    batch[key] = outputs[src]
            r = calc.forward(batch, model_params=model_params, state=state[name])
            new_state[name], outputs[name] = r["state"], r["output"]
        return {"state": new_state, "output": outputs}

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        out = {}
        for name, calc in self._calcs.items():
            sub = calc.get_summaries(model_params=model_params, state=state[name],
                                     all_forward_outputs=[o[name] for o in all_forward_outputs])
            for k, v in flatten_items(sub, is_leaf=lambda x: isinstance(x, MetricSummary)):
                out[f"{name}/{k}"] = v
        return out


class PredictionOutputs(NamedTuple):
    input_batch: dict
    predict_outputs: Any


class GlobalMetricCalculator(BaseMetricCalculator):
    """Collects ``model.<predict_method>`` outputs of every eval batch (moved to host memory)
    and computes metrics over all of them at once with ``metric_fn(list[PredictionOutputs])``
    (e.g. ranking / retrieval metrics that are not sums over batches)."""

    @config_class
    class Config(BaseMetricCalculator.Config):
        predict_method: str = "predict"
        predict_input_field: Optional[str] = None
        metric_fn: Required[Callable] = REQUIRED

    def init_state(self, *, prng_key, model_params):
        return {"prng_key": prng_key}

    def forward(self, input_batch, *, model_params, state):
        cfg = self._config
        key, next_key = prng.split(state["prng_key"], 2)
        batch = input_batch[cfg.predict_input_field] if cfg.predict_input_field else input_batch
        outputs, _ = self._call_model(method=cfg.predict_method, prng_key=key, model_params=model_params,
                                      input_batch=batch)
        to_host = lambda t: t.detach().cpu() if isinstance(t, Tensor) else t
        return {"state": {"prng_key": next_key},
                "output": PredictionOutputs(tree_map(to_host, input_batch), tree_map(to_host, outputs))}

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        metrics = self._config.metric_fn(all_forward_outputs)
        return {k: (v if isinstance(v, MetricSummary) else WeightedSummary(torch.as_tensor(v), 1))
                for k, v in metrics.items()}


class SpmdEvaler(Module):
    @config_class
    class Config(Module.Config):
        input: Required[InstantiableConfig] = REQUIRED
        summary_writer: InstantiableConfig = SummaryWriter.default_config()
        eval_policy: InstantiableConfig = config_for_function(every_n_steps_policy)
        eval_dtype: Optional[torch.dtype] = None
        metric_calculator: InstantiableConfig = ModelSummaryAccumulator.default_config()
        # Cap on the number of batches per evaluation (None = the whole eval input).
        max_batches: Optional[int] = None
        dir: Optional[str] = None
        # Batch indices at which a profiler trace of ONE forward is written under
        # ``{summary dir}/traces`` (at most three evaluations are traced, so that a long run does
        # not fill the disk; reference: axlearn/common/evaler.py:577, :699).
        trace_at_iters: Sequence[int] = ()
        # Writes every batch's inputs and per-example outputs (e.g. ``JsonlOutputWriter``).
        output_writer: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None, model=None, model_param_partition_specs=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        self._allow_contextless = True
        base = cfg.dir or (getattr(parent.config, "dir", None) if parent is not None else None) or "."
        sw = cfg.summary_writer.clone()
        if not getattr(sw, "dir", None):
            sw.dir = os.path.join(base, "summaries", cfg.name or "eval")
        self._add_child("input", maybe_set_config(cfg.input.clone(), is_training=False))
        self._add_child("metric_calculator", cfg.metric_calculator.clone(eval_dtype=cfg.eval_dtype), model=model,
                        model_param_partition_specs=model_param_partition_specs)
        self._add_child("summary_writer", sw)
        if cfg.output_writer is not None:
            self._add_child("output_writer", cfg.output_writer)
        self._trace_dir = os.path.join(sw.dir, "traces")
        self._traced_evals = 0
        self._policy: EvalPolicy = cfg.eval_policy.instantiate()
        self.last_eval_seconds: Optional[float] = None

    def eval_step(self, step: int, *, prng_key: Tensor, model_params: Any, return_aux: bool = False,
                  train_summaries: Optional[dict] = None, force_run: bool = False):
        """Returns ``(prng_key, summaries or None, per-batch outputs or None)``."""
        if not force_run and not self._policy(step=step, train_summaries=train_summaries or {}):
            return prng_key, None, None
        cfg = self._config
        t0 = time.perf_counter()
        prng_key, eval_key = prng.split(prng_key, 2)
        calc = self.metric_calculator
        state = calc.init_state(prng_key=eval_key, model_params=model_params)
        outputs = []
        traced_any = False
        device = next((t.device for _, t in flatten_items(model_params) if isinstance(t, Tensor)), None)
        for i, batch in enumerate(self.input.batches(iter(self.input.dataset()))):
            if cfg.max_batches is not None and i >= cfg.max_batches:
                break
            batch = tree_map(lambda t: t.to(device) if isinstance(t, Tensor) and device is not None else t, batch)
            if i in cfg.trace_at_iters and self._traced_evals < 3:
                traced_any = True
                r = self._traced_forward(calc, batch, model_params, state, step=step, batch_index=i)
            else:
                r = calc.forward(batch, model_params=model_params, state=state)
            state = r["state"]
            if return_aux or isinstance(calc, (GlobalMetricCalculator, CompositeMetricCalculator)):
                outputs.append(r["output"])
            if "output_writer" in self._children:
                self.output_writer.write(input_batch=batch, output_batch=r["output"])
        if traced_any:
            self._traced_evals += 1
        if "output_writer" in self._children:
            self.output_writer.flush()
        summaries = calc.get_summaries(model_params=model_params, state=state, all_forward_outputs=outputs)
        self.last_eval_seconds = time.perf_counter() - t0
        self.summary_writer(step, {**summaries, "eval_time_secs": self.last_eval_seconds})
        return prng_key, summaries, (outputs if return_aux else None)

    def _traced_forward(self, calc, batch, model_params, state, *, step: int, batch_index: int):
        """One forward under the torch profiler; the Chrome trace lands in ``traces/``."""
        from torch.profiler import ProfilerActivity, profile

        activities = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        os.makedirs(self._trace_dir, exist_ok=True)
        with profile(activities=activities) as prof:
            r = calc.forward(batch, model_params=model_params, state=state)
            if torch.cuda.is_available():
                torch.cuda.synchronize()
        prof.export_chrome_trace(os.path.join(self._trace_dir, f"eval_step{step:08d}_batch{batch_index}.json"))
        return r
