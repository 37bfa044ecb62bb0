"""Loading a trained model and running one of its methods over batches of inputs.

Parity targets in the reference: ``InferenceRunner`` (axlearn/common/inference.py:148-470:
mesh + model + ``init_state_builder`` that restores parameters; ``create_method_runner`` returns
a callable ``input_batch -> Output(prng_key, output_batch, summaries)``; ``run`` maps it over an
iterable), ``MethodRunner`` (:46), ``InferencePipeline`` (axlearn/common/inference_pipeline.py:83:
input -> runner -> output writer) and the JSON-lines output writer
(axlearn/common/inference_output.py:131-235).
"""

from __future__ import annotations

import json
import os
from typing import Any, Iterable, Iterator, NamedTuple, Optional, Sequence

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.module import Module, functional
from axlearn_b200.common.state_builder import Builder, TensorStoreStateStorageBuilder
from axlearn_b200.common.utils import TensorSpec, flatten_items, tree_map, unflatten_items
from axlearn_b200.parallel import collectives as coll
from axlearn_b200.parallel.mesh import create_mesh

Tensor = torch.Tensor


class MethodRunner:
    """``runner(input_batch) -> Output``; threads the PRNG key from call to call."""

    class Output(NamedTuple):
        prng_key: Tensor
        output_batch: Any
        summaries: dict

    def __init__(self, *, model, params, method: str, prng_key: Tensor, device, dtype=None, mesh=None,
                 drop_module_outputs: bool = True):
        self._model, self._params, self._method = model, params, method
        self._key, self._device, self._dtype, self._mesh = prng_key, device, dtype, mesh
        self._drop = ("module_outputs",) if drop_module_outputs else ()

    def __call__(self, input_batch: dict) -> "MethodRunner.Output":
        key, self._key = prng.split(self._key, 2)

        def place(t):
            if not isinstance(t, Tensor):
                return t
            t = t.to(self._device)
            return t.to(self._dtype) if self._dtype is not None and t.is_floating_point() else t

        batch = tree_map(place, input_batch)
        with torch.no_grad():
            if self._mesh is not None:
                with self._mesh:
                    out, oc = functional(self._model, key, self._params, dict(input_batch=batch), is_training=False,
                                         method=self._method, drop_output_collections=self._drop)
            else:
                out, oc = functional(self._model, key, self._params, dict(input_batch=batch), is_training=False,
                                     method=self._method, drop_output_collections=self._drop)
        return MethodRunner.Output(prng_key=self._key, output_batch=out, summaries=oc.summaries)


class InferenceRunner(Module):
    @config_class
    class Config(Module.Config):
        mesh_shape: Sequence[int] = (1,)
        mesh_axis_names: Sequence[str] = ("data",)
        model: Required[InstantiableConfig] = REQUIRED
        # Restores the parameters; by default from a checkpoint directory (set ``.dir``).
        init_state_builder: InstantiableConfig = TensorStoreStateStorageBuilder.default_config().set(
            include=r"model/.*")
        inference_dtype: Optional[torch.dtype] = None
        device: Optional[str] = None

    @classmethod
    def config_from_trainer(cls, trainer_cfg) -> "InferenceRunner.Config":
        return cls.default_config().set(
            name=trainer_cfg.name, mesh_shape=trainer_cfg.mesh_shape, mesh_axis_names=trainer_cfg.mesh_axis_names,
            model=trainer_cfg.model)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True
        cfg = self._config
        self._device = torch.device(cfg.device) if cfg.device else (
            torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available()
            else torch.device("cpu"))
        self._mesh = create_mesh(cfg.mesh_shape, cfg.mesh_axis_names) if coll.process_count() > 1 else None
        self._add_child("model", cfg.model.clone(name=cfg.model.name or "model"))
        self._add_child("init_state_builder", cfg.init_state_builder)
        specs = self.model.create_parameter_specs_recursively()
        structure = {"model": tree_map(
            lambda s: TensorSpec(shape=tuple(s.shape), dtype=s.dtype or torch.float32), specs,
            is_leaf=lambda x: hasattr(x, "mesh_axes"))}
        built = self.init_state_builder(Builder.State(step=0, trainer_state=structure, built_keys=set()))
        missing = [p for p, v in flatten_items(built.trainer_state) if not isinstance(v, Tensor)]
        if missing:
            raise ValueError(f"the state builder did not provide {len(missing)} parameters, e.g. {missing[:3]}")
        dtype = cfg.inference_dtype

        def place(t):
            t = t.to(self._device)
            return t.to(dtype) if dtype is not None and t.is_floating_point() else t

        self._params = tree_map(place, built.trainer_state["model"])
        self.step = built.step

    @property
    def model_params(self):
        return self._params

    def create_method_runner(self, *, method: str, prng_key: Optional[Tensor] = None,
                             drop_module_outputs: bool = True) -> MethodRunner:
        return MethodRunner(model=self.model, params=self._params, method=method,
                            prng_key=prng_key if prng_key is not None else prng.PRNGKey(0), device=self._device,
                            dtype=self._config.inference_dtype, mesh=self._mesh,
                            drop_module_outputs=drop_module_outputs)

    def run(self, input_batches: Iterable[dict], *, method: str, prng_key: Optional[Tensor] = None) -> Iterator[dict]:
        """Yields ``{"inputs": batch, "outputs": method(batch)}`` per input batch."""
        runner = self.create_method_runner(method=method, prng_key=prng_key)
        for batch in input_batches:
            out = runner(batch)
            yield {"inputs": batch, "outputs": out.output_batch}


class JsonlOutputWriter(Module):
    """One JSON object per example: ``{path: value}`` of the (optionally filtered) input and
    output leaves; one file per process (``name-{process:05d}-of-{count:05d}.jsonl``)."""

    @config_class
    class Config(Module.Config):
        output_dir: Required[str] = REQUIRED
        file_name: str = "outputs"
        include_inputs: bool = True
        output_keys: Optional[Sequence[str]] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True
        os.makedirs(cfg.output_dir, exist_ok=True)
        path = os.path.join(cfg.output_dir,
                            f"{cfg.file_name}-{coll.process_index():05d}-of-{coll.process_count():05d}.jsonl")
        self.path = path
        self._f = open(path, "w", encoding="utf-8")  # pylint: disable=consider-using-with

    def write(self, *, input_batch: dict, output_batch: Any) -> None:
        cfg = self._config
        flat = {}
        if cfg.include_inputs:
            flat.update({f"inputs/{k}": v for k, v in flatten_items(input_batch)})
        outs = output_batch if isinstance(output_batch, dict) else {"output": output_batch}
        flat.update({k: v for k, v in flatten_items(outs) if cfg.output_keys is None or k in cfg.output_keys})
        flat = {k: v for k, v in flat.items() if isinstance(v, Tensor) and v.dim() >= 1}
        if not flat:
            return
        n = next(iter(flat.values())).shape[0]
        for i in range(n):
            rec = {k: v[i].detach().float().cpu().tolist() if v.is_floating_point() else v[i].detach().cpu().tolist()
                   for k, v in flat.items() if v.shape[0] == n}
            self._f.write(json.dumps(rec) + "\n")

    def flush(self) -> None:
        self._f.flush()

    def close(self) -> None:
        self._f.close()


class InferencePipeline(Module):
    """input -> ``runner.<model_method>`` -> output writer."""

    @config_class
    class Config(Module.Config):
        input: Required[InstantiableConfig] = REQUIRED
        runner: Required[InstantiableConfig] = REQUIRED
        output_writer: Required[InstantiableConfig] = REQUIRED
        model_method: str = "predict"
        summary_writer: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True
        self._add_child("input", cfg.input)
        self._add_child("runner", cfg.runner)
        self._add_child("output_writer", cfg.output_writer)

    def run(self, *, prng_key: Optional[Tensor] = None) -> int:
        """Returns the number of batches processed."""
        n = 0
        for rec in self.runner.run(self.input.batches(iter(self.input.dataset())), method=self._config.model_method,
                                   prng_key=prng_key):
            self.output_writer.write(input_batch=rec["inputs"], output_batch=rec["outputs"])
            n += 1
        self.output_writer.flush()
        return n
