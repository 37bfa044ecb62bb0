"""Windowed self-attention for large feature maps (ViTDet): attention inside non-overlapping
windows of the patch grid, with a few global-attention layers in between.

Reference: axlearn/vision/window_attention.py (``window_partition_with_window_size`` :20,
``window_unpartition_with_window_size`` :65, ``WindowedAttention`` :105-174) and
axlearn/vision/vitdet_transformer.py (the stack that alternates windowed and global blocks).
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from axlearn_b200.common.attention import TransformerLayer
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class

Tensor = torch.Tensor


def window_partition(x: Tensor, window_size: int) -> tuple[Tensor, tuple[int, int]]:
    """``[B, H, W, C] -> [B * windows, window_size, window_size, C]`` (zero padding on the bottom
    and right when the grid is not a multiple) and the padded ``(H, W)``."""
    b, h, w, c = x.shape
    ph, pw = (-h) % window_size, (-w) % window_size
    if ph or pw:
        x = F.pad(x, (0, 0, 0, pw, 0, ph))
    hp, wp = h + ph, w + pw
    x = x.reshape(b, hp // window_size, window_size, wp // window_size, window_size, c)
    return x.permute(0, 1, 3, 2, 4, 5).reshape(-1, window_size, window_size, c), (hp, wp)


def window_unpartition(windows: Tensor, window_size: int, padded_hw: tuple[int, int], hw: tuple[int, int]) -> Tensor:
    hp, wp = padded_hw
    b = windows.shape[0] // ((hp // window_size) * (wp // window_size))
    x = windows.reshape(b, hp // window_size, wp // window_size, window_size, window_size, -1)
    x = x.permute(0, 1, 3, 2, 4, 5).reshape(b, hp, wp, -1)
    return x[:, :hw[0], :hw[1]]


class WindowedTransformerLayer(BaseLayer):
    """A transformer layer applied inside windows of a ``[B, H, W, C]`` map (``window_size=0``:
    global attention over the whole map).  Padding cells are masked out of the attention."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        window_size: int = 14
        layer: InstantiableConfig = TransformerLayer.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("layer", cfg.layer.clone(input_dim=cfg.input_dim))

    def forward(self, x: Tensor) -> Tensor:
        ws = self._config.window_size
        b, h, w, c = x.shape
        if not ws:
            return self.layer(x.reshape(b, h * w, c)).data.reshape(b, h, w, c)
        windows, padded = window_partition(x, ws)
        bias = None
        if padded != (h, w):
            live, _ = window_partition(torch.ones(1, h, w, 1, device=x.device), ws)
            live = live.reshape(-1, ws * ws).repeat(b, 1) > 0
            bias = torch.where(live[:, None, None, :], 0.0, -1e9).to(x.dtype)
        y = self.layer(windows.reshape(-1, ws * ws, c), self_attention_logit_biases=bias).data
        return window_unpartition(y.reshape(-1, ws, ws, c), ws, padded, (h, w))


class ViTDetTransformer(BaseLayer):
    """``num_layers`` blocks over a patch grid; blocks listed in ``global_attention_indices`` see
    the whole map, the others attend inside windows."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_layers: Required[int] = REQUIRED
        window_size: int = 14
        global_attention_indices: Optional[Sequence[int]] = None     # default: every fourth block
        layer: InstantiableConfig = TransformerLayer.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        glob = cfg.global_attention_indices
        if glob is None:
            step = max(1, cfg.num_layers // 4)
            glob = [i for i in range(cfg.num_layers) if (i + 1) % step == 0]
        self._global = set(glob)
        for i in range(cfg.num_layers):
            self._add_child(f"layer{i}", WindowedTransformerLayer.default_config().set(
                input_dim=cfg.input_dim, window_size=0 if i in self._global else cfg.window_size, layer=cfg.layer.clone()))

    def forward(self, x: Tensor) -> Tensor:
        for i in range(self._config.num_layers):
            x = getattr(self, f"layer{i}")(x)
        return x
