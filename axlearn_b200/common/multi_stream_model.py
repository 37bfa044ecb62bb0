"""Multi-tower and cross-encoder models as stream encoders plus fusion networks.

Reference: axlearn/common/multi_stream_model.py (``StreamEncoder`` :42, ``FusionNetwork`` :67,
``MultiStreamModel`` :99-213).  Every stream encoder adds its outputs to the batch under its own
name; every fusion network reads the batch and returns ``(loss, outputs)``; the model's loss is
the weighted sum of the fusion losses.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Any

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import InstantiableConfig, config_class


class StreamEncoder(BaseLayer):
    """``forward(input_batch) -> dict`` of encoded features."""

    def forward(self, input_batch: dict) -> dict:
        raise NotImplementedError(type(self))


class FusionNetwork(BaseLayer):
    """``forward(input_batch) -> (loss, outputs)`` over the stream encoders' features."""

    def forward(self, input_batch: dict) -> tuple[torch.Tensor, dict]:
        raise NotImplementedError(type(self))


class MultiStreamModel(BaseModel):
    @config_class
    class Config(BaseModel.Config):
        # Names of stream encoders and fusion networks must not collide.
        stream_encoder: dict[str, InstantiableConfig] = {}
        fusion_network: dict[str, InstantiableConfig] = {}
        loss_weights: dict[str, float] = {}          # default weight 1

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        names = list(cfg.stream_encoder) + list(cfg.fusion_network)
        if len(names) != len(set(names)):
            raise ValueError(f"duplicate stream / fusion names: {names}")
        self._stream_encoder = {n: self._add_child(n, self._overwrite_config(n, c))
                                for n, c in cfg.stream_encoder.items()}
        self._fusion_network = {n: self._add_child(n, self._overwrite_config(n, c))
                                for n, c in cfg.fusion_network.items()}

    def _overwrite_config(self, child_name: str, child_config: InstantiableConfig) -> InstantiableConfig:
        """Hook for subclasses to adjust a child's config."""
        del child_name
        return child_config

    def _aggregate_loss(self, losses: dict[str, torch.Tensor]) -> torch.Tensor:
        weights = defaultdict(lambda: 1.0, self._config.loss_weights)
        return sum(losses[n] * weights[n] for n in self._fusion_network)

    def _forward_all_stream_encoder(self, input_batch: dict) -> dict:
        for name, enc in self._stream_encoder.items():
            if name in input_batch:
                raise ValueError(f"{name} is already a key of the batch")
            input_batch[name] = enc(input_batch["input"])
        return input_batch

    def forward_single_stream_encoder(self, input_batch: dict, encoder_name: str) -> Any:
        """Runs one tower (the entry point for offline embedding extraction)."""
        if encoder_name not in self._stream_encoder:
            raise ValueError(f"{encoder_name} is not a stream encoder")
        return self._stream_encoder[encoder_name](input_batch["input"])

    def predict(self, input_batch: dict) -> dict:
        return self._forward_all_stream_encoder(dict(input_batch))

    def forward(self, input_batch: dict) -> tuple[torch.Tensor, dict]:
        input_batch = self._forward_all_stream_encoder(dict(input_batch))
        losses = {}
        for name, net in self._fusion_network.items():
            if name in input_batch:
                raise ValueError(f"{name} is already a key of the batch")
            loss, input_batch[name] = net(input_batch)
            self.add_summary(f"loss_{name}", loss)
            losses[name] = loss
        return self._aggregate_loss(losses), {}
