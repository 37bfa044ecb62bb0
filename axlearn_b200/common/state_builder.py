"""Builders that produce (parts of) a trainer state from elsewhere: checkpoints of other runs,
converted parameter trees, modified weights.

Parity targets in the reference (axlearn/common/state_builder.py): ``Builder`` (:54) with
``input_state_type`` / ``__call__(State)``, ``ChainBuilder`` (:95), ``Converter`` (:138),
``ChainConverter`` (:183), ``MergeStateConverter`` (:245), ``RestoreAndConvertBuilder`` (:298),
``TensorStoreStateStorageBuilder`` (:392: load a checkpoint directory into the state),
``ModelStateScopeConverter`` (:554: copy sub-trees between scopes), ``EmaParamsConverter`` (:767)
and ``get_builder`` (:1005).

A ``Builder.State`` is ``(step, trainer_state, built_keys)``: ``trainer_state`` is the nested dict
the trainer owns and ``built_keys`` the set of tensor paths that are already final (the trainer
initialises the rest).  Used as ``SpmdTrainer.Config.init_state_builder``: the trainer asks
``prebuilt_model_params(trainer)`` before initialising parameters.
"""

from __future__ import annotations

import enum
import os
import re
from typing import Any, NamedTuple, Optional, Sequence, Union

import torch

from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.module import Module
from axlearn_b200.common.utils import flatten_items, tree_map, unflatten_items

Tensor = torch.Tensor


class Builder(Module):
    class StateType(enum.Enum):
        TENSORS = "tensors"           # needs a fully initialised state as input
        TENSOR_SPECS = "tensor_specs" # only needs the structure (shapes / dtypes)

    class State(NamedTuple):
        step: int
        trainer_state: Any
        built_keys: set

    @config_class
    class Config(Module.Config):
        pass

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True

    def input_state_type(self) -> "Builder.StateType":
        raise NotImplementedError(type(self))

    def __call__(self, state: "Builder.State") -> "Builder.State":
        raise NotImplementedError(type(self))

    # Trainer hook: the model-parameter sub-tree this builder provides (paths relative to the
    # model), or None.
    def prebuilt_model_params(self, trainer) -> Optional[dict]:
        structure = trainer._state_structure()  # pylint: disable=protected-access
        out = self(Builder.State(step=0, trainer_state=structure, built_keys=set()))
        prefix = "model/"
        items = [(k[len(prefix):], v) for k, v in flatten_items(out.trainer_state)
                 if k in out.built_keys and k.startswith(prefix) and isinstance(v, Tensor)]
        return unflatten_items(items) if items else None


class ChainBuilder(Builder):
    """Applies builders in order; TENSOR_SPECS builders must come before TENSORS builders."""

    @config_class
    class Config(Builder.Config):
        builders: Required[Sequence[InstantiableConfig]] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._builders = [self._add_child(f"builder{i:03d}", b) for i, b in enumerate(cfg.builders)]
        seen_tensors = False
        for b in self._builders:
            t = b.input_state_type()
            if t == Builder.StateType.TENSORS:
                seen_tensors = True
            elif seen_tensors:
                raise ValueError("a TENSOR_SPECS builder cannot follow a TENSORS builder")

    def input_state_type(self):
        return self._builders[0].input_state_type()

    def __call__(self, state):
        for b in self._builders:
            state = b(state)
        return state


class Converter(Module):
    """Maps between the state layout of the current model and that of a source checkpoint:
    ``target_to_source`` builds the structure to restore into, ``source_to_target`` puts the
    restored tensors where the target wants them."""

    @config_class
    class Config(Module.Config):
        pass

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True

    def target_state_type(self) -> Builder.StateType:
        return Builder.StateType.TENSOR_SPECS

    def target_to_source(self, target: Builder.State) -> tuple[Builder.State, Any]:
        return target, None

    def source_to_target(self, source: Builder.State, aux: Any) -> Builder.State:
        return source


class ChainConverter(Converter):
    @config_class
    class Config(Converter.Config):
        converters: Required[Sequence[InstantiableConfig]] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._converters = [self._add_child(f"converter{i:03d}", c) for i, c in enumerate(cfg.converters)]

    def target_to_source(self, target):
        auxes = []
        for c in self._converters:
            target, aux = c.target_to_source(target)
            auxes.append(aux)
        return target, auxes

    def source_to_target(self, source, aux):
        for c, a in zip(reversed(self._converters), reversed(aux)):
            source = c.source_to_target(source, a)
        return source


class ModelStateScopeConverter(Converter):
    """Copies sub-trees of the source model into scopes of the target model.

    ``scope``: ``{target_scope: source_scope}`` (paths with ``/``; ``""`` = the whole model), or a
    single string for "same scope on both sides".  Only the listed target scopes count as built.
    """

    @config_class
    class Config(Converter.Config):
        scope: Union[str, dict, None] = None

    def _scopes(self) -> dict:
        s = self._config.scope
        if s is None:
            return {"": ""}
        if isinstance(s, str):
            return {s: s}
        return dict(s)

    def target_to_source(self, target):
        model = target.trainer_state["model"]
        source_items = []
        for tgt_scope, src_scope in self._scopes().items():
            for path, v in flatten_items(_subtree(model, tgt_scope)):
                source_items.append((_join(src_scope, path), v))
        source_state = {"model": unflatten_items(source_items)}
        return Builder.State(step=target.step, trainer_state=source_state, built_keys=set()), target

    def source_to_target(self, source, aux):
        target: Builder.State = aux
        model_items = dict(flatten_items(target.trainer_state["model"]))
        built = set(target.built_keys)
        src_model = dict(flatten_items(source.trainer_state["model"]))
        for tgt_scope, src_scope in self._scopes().items():
            for path in [p for p in model_items if _in_scope(p, tgt_scope)]:
                rel = path[len(tgt_scope):].lstrip("/") if tgt_scope else path
                src_path = _join(src_scope, rel)
                if src_path in src_model and isinstance(src_model[src_path], Tensor):
                    model_items[path] = src_model[src_path]
                    built.add("model/" + path)
        state = dict(target.trainer_state)
        state["model"] = unflatten_items(list(model_items.items()))
        return Builder.State(step=target.step, trainer_state=state, built_keys=built)


def _join(scope: str, path: str) -> str:
    return f"{scope}/{path}" if scope and path else (scope or path)


def _in_scope(path: str, scope: str) -> bool:
    return not scope or path == scope or path.startswith(scope + "/")


def _subtree(tree: dict, scope: str):
    node = tree
    for part in [p for p in scope.split("/") if p]:
        node = node[part]
    return node


class TensorStoreStateStorageBuilder(Builder):
    """Restores tensors from a checkpoint directory (``.../checkpoints/step_XXXXXXXX``) into the
    state: every tensor whose path exists in the checkpoint with the same shape is loaded
    (validation ``CONTAINS_STATE_UP_TO_DTYPE`` in the reference's terms)."""

    @config_class
    class Config(Builder.Config):
        dir: Required[str] = REQUIRED
        # Regex on tensor paths to load (None = everything that matches by name).
        include: Optional[str] = None

    def input_state_type(self):
        return Builder.StateType.TENSOR_SPECS

    def __call__(self, state):
        from axlearn_b200.common.checkpointer import parse_step_from_dir, read_state_tensors

        cfg = self._config
        stored = read_state_tensors(cfg.dir)
        pat = re.compile(cfg.include) if cfg.include else None
        items, built = [], set(state.built_keys)
        for path, v in flatten_items(state.trainer_state):
            if path in stored and (pat is None or pat.fullmatch(path)):
                want = tuple(getattr(v, "shape", ()))
                t = stored[path]
                if tuple(t.shape) != want:
                    raise ValueError(f"{path}: checkpoint has shape {tuple(t.shape)}, the state wants {want}")
                dtype = getattr(v, "dtype", t.dtype)
                items.append((path, t.to(dtype)))
                built.add(path)
            else:
                items.append((path, v))
        try:
            step = parse_step_from_dir(cfg.dir)
        except Exception:  # pylint: disable=broad-except
            step = state.step
        return Builder.State(step=step, trainer_state=unflatten_items(items), built_keys=built)


class RestoreAndConvertBuilder(Builder):
    """``converter.target_to_source`` -> restore with ``builder`` -> ``converter.source_to_target``:
    initialise (part of) a model from a checkpoint of a differently-structured model."""

    @config_class
    class Config(Builder.Config):
        builder: Required[InstantiableConfig] = REQUIRED
        converter: Required[InstantiableConfig] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("builder", cfg.builder)
        self._add_child("converter", cfg.converter)

    def input_state_type(self):
        return self.converter.target_state_type()

    def __call__(self, state):
        source, aux = self.converter.target_to_source(state)
        restored = self.builder(source)
        return self.converter.source_to_target(restored, aux)


class EmaParamsConverter(Converter):
    """Loads the EMA weights of the source (``learner/ema/ema/...``) as the target's model
    parameters."""

    def target_to_source(self, target):
        model = target.trainer_state["model"]
        source = {"learner": {"ema": {"ema": model}}}
        return Builder.State(step=target.step, trainer_state=source, built_keys=set()), target

    def source_to_target(self, source, aux):
        target: Builder.State = aux
        ema = source.trainer_state["learner"]["ema"]["ema"]
        state = dict(target.trainer_state)
        state["model"] = ema
        built = set(target.built_keys) | {
            "model/" + p for p, v in flatten_items(ema) if isinstance(v, Tensor)}
        return Builder.State(step=target.step, trainer_state=state, built_keys=built)


class SimpleWeightModifierBuilder(Builder):
    """Applies ``modify(path, tensor) -> tensor`` to the model parameters whose path matches."""

    @config_class
    class Config(Builder.Config):
        path_regex: str = ".*"
        modify: Required[Any] = REQUIRED

    def input_state_type(self):
        return Builder.StateType.TENSORS

    def __call__(self, state):
        pat = re.compile(self._config.path_regex)
        items = []
        for path, v in flatten_items(state.trainer_state):
            if isinstance(v, Tensor) and path.startswith("model/") and pat.fullmatch(path[len("model/"):]):
                v = self._config.modify(path, v)
            items.append((path, v))
        return Builder.State(step=state.step, trainer_state=unflatten_items(items), built_keys=state.built_keys)


def get_builder_config(spec: Union[str, InstantiableConfig]) -> InstantiableConfig:
    """A builder config from a spec string: a checkpoint directory becomes a
    ``TensorStoreStateStorageBuilder``."""
    if isinstance(spec, InstantiableConfig):
        return spec
    if isinstance(spec, str) and os.path.basename(spec.rstrip("/")).startswith("step_"):
        return TensorStoreStateStorageBuilder.default_config().set(dir=spec)
    raise NotImplementedError(f"no builder understands the spec {spec!r}")
