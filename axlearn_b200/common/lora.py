"""Low-rank adapters for linear and fused-QKV layers.

Parity targets in the reference (axlearn/common/lora.py): ``LoraLinear`` (child ``layer`` = the
frozen base ``Linear``, children ``lora_down`` ``[in, rank]`` and ``lora_up`` ``[rank, out]``,
output ``base(x) + alpha / rank * up(down(dropout(x)))``, ``lora_up`` initialised to zero) and
``LoraFusedQKVLinear`` (adapters on a chosen subset of q / k / v).
"""

from __future__ import annotations

from typing import Sequence

import torch

from axlearn_b200.common.attention import BaseQKVLinear, FusedQKVLinear
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Dropout, Linear
from axlearn_b200.common.param_init import ConstantInitializer, DefaultInitializer

Tensor = torch.Tensor


def _zero_weight_init():
    return DefaultInitializer.default_config().set(
        init_by_param_name={".*weight$": ConstantInitializer.default_config().set(value=0.0)})


class _LoraAdapter(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        rank: Required[int] = REQUIRED
        alpha: Required[float] = REQUIRED
        dropout: InstantiableConfig = Dropout.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("lora_down", Linear.default_config().set(
            input_dim=cfg.input_dim, output_dim=cfg.rank, bias=False, param_partition_spec=(None, None)))
        self._add_child("lora_up", Linear.default_config().set(
            input_dim=cfg.rank, output_dim=cfg.output_dim, bias=False, param_partition_spec=(None, None),
            param_init=_zero_weight_init()))
        self._add_child("dropout", cfg.dropout)

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        return self.lora_up(self.lora_down(self.dropout(x))) * (cfg.alpha / cfg.rank)


class LoraLinear(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        layer: InstantiableConfig = Linear.default_config()
        adapter: InstantiableConfig = _LoraAdapter.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("layer", cfg.layer.clone(input_dim=cfg.input_dim, output_dim=cfg.output_dim))
        self._add_child("adapter", cfg.adapter.clone(input_dim=cfg.input_dim, output_dim=cfg.output_dim))

    def forward(self, x: Tensor) -> Tensor:
        return self.layer(x) + self.adapter(x).to(x.dtype)


class LoraFusedQKVLinear(BaseQKVLinear):
    """Fused QKV projection plus adapters on ``enable_lora`` of ("query", "key", "value")."""

    @config_class
    class Config(BaseQKVLinear.Config):
        layer: InstantiableConfig = FusedQKVLinear.default_config()
        adapter: InstantiableConfig = _LoraAdapter.default_config()
        enable_lora: Sequence[str] = ("query", "value")

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("layer", cfg.layer.clone(
            query_dim=cfg.query_dim, key_dim=cfg.key_dim, value_dim=cfg.value_dim, num_heads=cfg.num_heads,
            per_head_dim=cfg.per_head_dim))
        for name in cfg.enable_lora:
            self._add_child(f"adapter_{name}", cfg.adapter.clone(
                input_dim=cfg.query_dim, output_dim=cfg.num_heads * cfg.per_head_dim))

    def forward(self, query: Tensor, *, key=None, value=None, kv_state=None, query_positions=None):
        cfg = self._config
        out = self.layer(query, key=key, value=value, kv_state=kv_state, query_positions=query_positions)
        parts = {"query": out.query, "key": out.key, "value": out.value}
        for name in cfg.enable_lora:
            delta = getattr(self, f"adapter_{name}")(query)
            parts[name] = parts[name] + delta.reshape(parts[name].shape).to(parts[name].dtype)
        return self.Output(parts["query"], parts["key"], parts["value"])
