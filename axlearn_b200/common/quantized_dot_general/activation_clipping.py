"""Activation clipping for int8 contractions (reference:
axlearn/common/quantized_dot_general/activation_clipping.py:19-186).

Symmetric int8 quantisation spends its 255 levels on ``[-max|x|, max|x|]``; one outlier makes
every other value coarse.  A clipping layer bounds the range first: hard (clamp), soft (tanh) or
not at all (summary only).  With ``clipping_summary`` each layer reports the fraction of values
outside the range as ``activations/clipped_activation``.
"""

from __future__ import annotations

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, Required, config_class

Tensor = torch.Tensor


class BaseActivationClippingLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        clipping_summary: bool = False

    def _maybe_add_clipping_summary(self, x: Tensor, clipping_max_abs) -> None:
        if self._config.clipping_summary:
            outside = (x.detach().abs() > clipping_max_abs).float().mean()
            self.add_summary("activations/clipped_activation", outside)

    def forward(self, x: Tensor) -> Tensor:
        raise NotImplementedError(type(self))


class _BoundedClippingLayer(BaseActivationClippingLayer):
    @config_class
    class Config(BaseActivationClippingLayer.Config):
        # Largest absolute value after clipping (the range is symmetric, as the quantiser's).
        clipping_max_abs: Required[float] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        bound = self._config.clipping_max_abs
        if bound is None or bound is REQUIRED or bound <= 0:
            raise ValueError(f"clipping_max_abs must be a positive float for {self.path()}. Found {bound}")


class HardActivationClippingLayer(_BoundedClippingLayer):
    """``clamp(x, -b, b)``; the gradient of clipped values is zero."""

    def forward(self, x: Tensor) -> Tensor:
        b = self._config.clipping_max_abs
        self._maybe_add_clipping_summary(x, b)
        return x.clamp(-b, b)


class DummyActivationClippingLayer(_BoundedClippingLayer):
    """Does not clip; only reports how much a hard clip at the bound would cut."""

    def forward(self, x: Tensor) -> Tensor:
        self._maybe_add_clipping_summary(x, self._config.clipping_max_abs)
        return x


class TanhActivationClippingLayer(_BoundedClippingLayer):
    """``b * tanh(x / b)``: the identity near zero, saturating smoothly at the bound."""

    def forward(self, x: Tensor) -> Tensor:
        b = self._config.clipping_max_abs
        self._maybe_add_clipping_summary(x, b)
        return torch.tanh(x / b) * b
