"""B200-native training and serving framework with the public surface of AXLearn.

``import axlearn_b200 as ax`` gives the commonly used names lazily (``ax.config_class``,
``ax.BaseModel``, ``ax.layers.Linear``, ``ax.SpmdTrainer`` ...); nothing heavy is imported until
an attribute is first used.
"""

import importlib
from typing import Any

_MODULES = {
    name: f"axlearn_b200.common.{name}"
    for name in (
        "attention", "base_layer", "base_model", "causal_lm", "checkpointer", "config", "decoder", "decoding",
        "embedding", "evaler", "input_base", "input_fake", "input_lm", "input_pipeline", "layers", "learner",
        "loss", "metrics", "module", "optimizers", "param_init", "prng", "schedule", "state_builder",
        "summary_writer", "trainer", "utils",
    )
}
_NAMES = {
    "BaseLayer": ("base_layer", "BaseLayer"),
    "ParameterSpec": ("base_layer", "ParameterSpec"),
    "BaseModel": ("base_model", "BaseModel"),
    "Module": ("module", "Module"),
    "functional": ("module", "functional"),
    "SpmdTrainer": ("trainer", "SpmdTrainer"),
    "config_class": ("config", "config_class"),
    "config_for_function": ("config", "config_for_function"),
    "config_for_class": ("config", "config_for_class"),
    "REQUIRED": ("config", "REQUIRED"),
    "Required": ("config", "Required"),
    "InstantiableConfig": ("config", "InstantiableConfig"),
}


def __getattr__(name: str) -> Any:
    if name in _MODULES:
        return importlib.import_module(_MODULES[name])
    if name in _NAMES:
        mod, attr = _NAMES[name]
        return getattr(importlib.import_module(_MODULES[mod]), attr)
    raise AttributeError(f"module 'axlearn_b200' has no attribute {name!r}")


def __dir__():
    return sorted(list(_MODULES) + list(_NAMES))
