"""Runs any ``torch.nn.Module`` as a layer of this framework.

Counterpart of axlearn/common/adapter_flax.py (``FlaxLayer`` :22-112, ``config_for_flax_module``
:115): the reference wraps modules of another layer library so that they take part in its
parameter trees, partitioning and checkpoints.  Here the foreign library is plain PyTorch: the
wrapped module's parameters and buffers become this layer's parameters (nested by their dotted
names), initialised from the module's own ``reset_parameters`` under the framework's seed, and the
forward pass is a ``torch.func.functional_call`` with the parameters of the current context, so
that gradients, sharded storage and checkpoints go through the framework, not through the module.
"""

from __future__ import annotations

from typing import Any, Callable, Optional

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.module import nowrap
from axlearn_b200.common.utils import flatten_items


class TorchModuleLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        # Zero-argument callable (or config) that builds the module.
        create_module_fn: Required[Callable[[], torch.nn.Module]] = REQUIRED
        create_module_kwargs: dict = {}
        # Mesh axes by parameter name (dotted); parameters not listed are replicated.
        mesh_axes_by_name: dict = {}

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._module = self._build()
        for p in self._module.parameters():
            p.requires_grad_(False)          # the framework's copies are the trainable ones

    def _build(self) -> torch.nn.Module:
        cfg = self._config
        return cfg.create_module_fn(**cfg.create_module_kwargs)

    @staticmethod
    def _nest(flat: dict) -> dict:
        out: dict = {}
        for name, value in flat.items():
            node = out
            *head, last = name.split(".")
            for k in head:
                node = node.setdefault(k, {})
            node[last] = value
        return out

    def _named_tensors(self, module: torch.nn.Module) -> dict:
        return {**dict(module.named_parameters()), **dict(module.named_buffers())}

    def _create_layer_parameter_specs(self):
        cfg = self._config
        specs = {}
        for name, t in self._named_tensors(self._module).items():
            specs[name] = ParameterSpec(shape=tuple(t.shape), dtype=t.dtype,
                                        mesh_axes=cfg.mesh_axes_by_name.get(name, (None,) * t.dim()))
        return self._nest(specs)

    @nowrap
    def create_parameter_specs_recursively(self):
        return self._create_layer_parameter_specs()

    @nowrap
    def initialize_parameters_recursively(self, prng_key, *, prebuilt=None, device="cpu"):
        """Initial values are the module's own, drawn under a seed derived from ``prng_key``."""
        seed = int(prng.randint(prng_key, (), 0, 2 ** 31 - 1))
        with torch.random.fork_rng(devices=[]):
            torch.manual_seed(seed)
            fresh = self._build()
        return self._nest({k: v.detach().clone().to(device) for k, v in self._named_tensors(fresh).items()})

    def forward(self, *args, **kwargs) -> Any:
        buffers = {name for name, _ in self._module.named_buffers()}
        flat = {}
        for path, t in flatten_items(self.state):
            name = path.replace("/", ".")
            flat[name] = t.detach() if name in buffers else t       # statistics carry no gradient
        self._module.train(self.is_training)
        return torch.func.functional_call(self._module, flat, args, kwargs)


def config_for_torch_module(create_module_fn: Callable[..., torch.nn.Module], **create_module_kwargs):
    return TorchModuleLayer.default_config().set(create_module_fn=create_module_fn, create_module_kwargs=create_module_kwargs)
