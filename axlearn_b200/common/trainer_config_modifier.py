"""Config modifiers: callables that rewrite a trainer config for a hardware target.

Parity targets in the reference (axlearn/common/trainer_config_modifier.py):
``GradientAccumulationModifier`` (:39), ``RematSpecModifier`` (:85), ``MeshShapeModifier``
(:125), ``ModuleConfigModifier`` (:152), ``ReplaceLayerConfigModifier``,
``PartitionSpecModifier`` (:200), ``ChainConfigModifier`` (:300), ``FP8ConfigModifier``
(:339-371).  Mesh rules select them by ``--mesh_selector``.
"""

from __future__ import annotations

from typing import Any, Optional, Sequence, Union

from axlearn_b200.common.base_layer import RematSpec
from axlearn_b200.common.config import (
    REQUIRED,
    ConfigBase,
    ConfigModifier,
    InstantiableConfig,
    Required,
    config_class,
)
from axlearn_b200.common.utils import replace_layer_config_recursively
from axlearn_b200.parallel.mesh import HybridMeshShape, MeshShape


def _find(cfg: ConfigBase, dotted: str) -> ConfigBase:
    """Resolves ``a.b.c`` below ``cfg`` with a helpful error."""
    cur = cfg
    for part in dotted.split("."):
        if not isinstance(cur, ConfigBase) or part not in cur:
            raise ValueError(f"{part} is not found in {type(cur).__qualname__} while resolving {dotted}")
        cur = getattr(cur, part)
    return cur


class GradientAccumulationModifier(ConfigModifier):
    """Runs ``grad_acc_steps`` micro-batches per optimizer step."""

    @config_class
    class Config(ConfigModifier.Config):
        grad_acc_steps: Required[int] = REQUIRED
        metric_accumulator: Optional[InstantiableConfig] = None

    def __call__(self, cfg):
        """The reference wraps the learner's forward function in ``with_minibatch_steps``
        (axlearn/common/trainer_config_modifier.py:60-103); here the trainer owns the loop."""
        cfg.grad_accumulation_steps = self._config.grad_acc_steps
        return cfg


class RematSpecModifier(ConfigModifier):
    """Sets ``remat_spec`` of the modules named by dotted paths."""

    @config_class
    class Config(ConfigModifier.Config):
        remat_policies: Required[dict[str, RematSpec]] = REQUIRED

    def __call__(self, cfg):
        for path, spec in self._config.remat_policies.items():
            target = _find(cfg, path)
            if "remat_spec" not in target:
                raise ValueError(f"{path} has no remat_spec field")
            target.remat_spec = spec
        return cfg


class MeshShapeModifier(ConfigModifier):
    @config_class
    class Config(ConfigModifier.Config):
        mesh_shape: Optional[Union[MeshShape, HybridMeshShape]] = None

    def __call__(self, cfg):
        cfg.mesh_shape = self._config.mesh_shape
        return cfg


class ModuleConfigModifier(ConfigModifier):
    """Replaces whole sub-configs: ``{dotted path: new config}``."""

    @config_class
    class Config(ConfigModifier.Config):
        target_config: Optional[str] = None
        modification: Optional[InstantiableConfig] = None
        module_configs: dict[str, Any] = {}

    def __call__(self, cfg):
        c = self._config
        items = dict(c.module_configs)
        if c.target_config is not None:
            items[c.target_config] = c.modification
        for path, new in items.items():
            parts = path.split(".")
            parent = _find(cfg, ".".join(parts[:-1])) if len(parts) > 1 else cfg
            setattr(parent, parts[-1], new)
        return cfg


class ReplaceLayerConfigModifier(ConfigModifier):
    """Replaces every sub-config of class ``target_cls`` by ``source_config``."""

    @config_class
    class Config(ConfigModifier.Config):
        target_cls: Required[type] = REQUIRED
        source_config: Required[InstantiableConfig] = REQUIRED

    def __call__(self, cfg):
        replace_layer_config_recursively(cfg, target_cls=self._config.target_cls, source_config=self._config.source_config)
        return cfg


class PartitionSpecModifier(ConfigModifier):
    """Sets partition-spec fields: ``{dotted module path: {field: spec}}``."""

    @config_class
    class Config(ConfigModifier.Config):
        partition_specs: Required[dict[str, dict[str, Any]]] = REQUIRED

    def __call__(self, cfg):
        for path, fields in self._config.partition_specs.items():
            target = _find(cfg, path)
            for name, spec in fields.items():
                if name not in target:
                    raise ValueError(f"{name} is not a field of {path}")
                setattr(target, name, spec)
        return cfg


class OverrideConfigModifier(ConfigModifier):
    """Sets arbitrary leaf fields: ``{dotted path: value}``."""

    @config_class
    class Config(ConfigModifier.Config):
        overrides: dict[str, Any] = {}

    def __call__(self, cfg):
        for path, v in self._config.overrides.items():
            cfg.set_recursively(path.split("."), value=v)
        return cfg


class ChainConfigModifier(ConfigModifier):
    @config_class
    class Config(ConfigModifier.Config):
        config_modifiers: Required[Sequence[InstantiableConfig]] = REQUIRED

    def __init__(self, cfg):
        super().__init__(cfg)
        self._mods = [m.instantiate() for m in cfg.config_modifiers]

    def __call__(self, cfg):
        for m in self._mods:
            cfg = m(cfg)
        return cfg


class FP8ConfigModifier(ConfigModifier):
    """Turns on fp8 GEMMs for every dense layer (``quantized_dot_general`` child) and routes
    the scale / amax-history "gradients" through in-place overrides."""

    @config_class
    class Config(ConfigModifier.Config):
        fp8_amax_history_length: int = 128
        # "tensor" = per-tensor delayed scaling (the reference's scheme);
        # "block" = 1x128 activation / 128x128 weight scale blocks.
        scaling: str = "block"

    def __call__(self, cfg):
        from axlearn_b200.common.quantized_dot_general.layers import QuantizedDotGeneral

        def visit(c):
            if isinstance(c, ConfigBase):
                if "quantized_dot_general" in c:
                    c.quantized_dot_general = QuantizedDotGeneral.default_config().set(
                        fp8_amax_history_length=self._config.fp8_amax_history_length, scaling=self._config.scaling)
                for _, v in c.items():
                    visit(v)
            elif isinstance(c, (list, tuple)):
                for x in c:
                    visit(x)
            elif isinstance(c, dict):
                for x in c.values():
                    visit(x)

        visit(cfg.model)
        if self._config.scaling == "tensor":
            # The new scales and amax histories arrive as the "gradients" of those parameters:
            # they overwrite the parameters instead of going through the optimizer (reference:
            # axlearn/common/trainer_config_modifier.py:362-370).
            from axlearn_b200.common.quantized_dot_general.layers import get_all_fp8_param_names
            from axlearn_b200.common.update_transformation import OverrideInplaceUpdateTransformation

            cfg.learner.optimizer = OverrideInplaceUpdateTransformation.default_config().set(
                rules=[f".*/{name}" for name in get_all_fp8_param_names()], transformation=cfg.learner.optimizer)
        return cfg
