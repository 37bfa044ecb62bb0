"""BaseModel: the contract between a model and the trainer.

Parity target: ``BaseModel`` in the reference (axlearn/common/base_model.py:46-127):
``forward(input_batch) -> (loss, aux)``; ``predict`` is optional.
"""

from __future__ import annotations

from typing import Any

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import config_class


class BaseModel(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        pass

    def forward(self, input_batch: dict) -> tuple[torch.Tensor, Any]:
        """Returns ``(loss, aux_outputs)``; ``loss`` is a scalar to be minimised."""
        raise NotImplementedError(type(self))

    def predict(self, input_batch: dict) -> Any:
        raise NotImplementedError(type(self))
