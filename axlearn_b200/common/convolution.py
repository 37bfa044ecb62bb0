"""Convolution layers (channels-last activations, reference weight layouts).

Parity targets in the reference (axlearn/common/convolution.py): ``Conv1D`` (weight
``[window, in/groups, out]``), ``Conv2D`` (``[h, w, in/groups, out]``), ``Conv3D``,
``Conv2DTranspose``, ``Conv2DWith1DPadding`` (paddings propagated for sequence models),
``StackOverTime``; ``padding`` is ``"SAME"``, ``"VALID"``, ``"CAUSAL"`` or explicit
``((lo, hi), ...)``.  Activations are ``[batch, spatial..., channels]``; parameter names and
shapes are the reference's so checkpoints map one to one.  The contraction itself goes to
cuDNN through ``torch.nn.functional`` (convolutions are outside this build's hot paths).
"""

from __future__ import annotations

from typing import Optional, Sequence, Union

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_layer import BaseLayer, FactorizationSpec, FanAxes, ParameterSpec
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.module import nowrap

Tensor = torch.Tensor
Padding = Union[str, Sequence[tuple]]


def _explicit_padding(padding: Padding, window: Sequence[int], strides: Sequence[int],
                      dilation: Sequence[int]) -> list[tuple[int, int]]:
    """Explicit ``(lo, hi)`` per spatial dim (axlearn/common/convolution.py:119-217), with
    ``w`` the dilated window: SAME = ``((w - 1) // 2, w - 1 - (w - 1) // 2)`` whatever the stride,
    VALID = ``(0, 0)``, CAUSAL = ``(w - stride, stride - 1)`` on the first (time) dim and SAME on
    the others."""
    if not isinstance(padding, str):
        return [tuple(p) for p in padding]
    eff = [(w - 1) * d + 1 for w, d in zip(window, dilation)]

    def same(w):
        total = w - 1
        return (total // 2, total - total // 2)

    if padding == "VALID":
        return [(0, 0)] * len(eff)
    if padding == "SAME":
        return [same(w) for w in eff]
    if padding == "CAUSAL":
        return [(eff[0] - strides[0], strides[0] - 1)] + [same(w) for w in eff[1:]]
    raise NotImplementedError(padding)


conv_explicit_padding = _explicit_padding


def conv_output_length(length: int, *, window: int, stride: int, padding: tuple[int, int], dilation: int = 1) -> int:
    eff = (window - 1) * dilation + 1
    return (length + padding[0] + padding[1] - eff) // stride + 1


class _ConvND(BaseLayer):
    ND = 2

    @config_class
    class Config(BaseLayer.Config):
        window: Sequence[int] = (1, 1)
        strides: Sequence[int] = (1, 1)
        dilation: Optional[Sequence[int]] = None
        padding: Padding = "VALID"
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        bias: bool = True
        num_input_dim_groups: int = 1

    def _create_layer_parameter_specs(self):
        cfg = self._config
        nd = self.ND
        if cfg.input_dim % cfg.num_input_dim_groups or cfg.output_dim % cfg.num_input_dim_groups:
            raise ValueError("input_dim and output_dim must be divisible by num_input_dim_groups")
        params = {"weight": ParameterSpec(
            shape=tuple(cfg.window) + (cfg.input_dim // cfg.num_input_dim_groups, cfg.output_dim),
            mesh_axes=(None,) * nd + (None, "model"),
            factorization=FactorizationSpec(axes=(None,) * nd + ("row", "col")),
            fan_axes=FanAxes(in_axis=-2, out_axis=-1))}
        if cfg.bias:
            params["bias"] = ParameterSpec(shape=(cfg.output_dim,), mesh_axes=("model",))
        return params

    @nowrap
    def _pad(self) -> list[tuple[int, int]]:
        cfg = self._config
        dil = cfg.dilation or (1,) * self.ND
        return _explicit_padding(cfg.padding, cfg.window, cfg.strides, dil)

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        nd = self.ND
        dil = tuple(cfg.dilation or (1,) * nd)
        w = self.parameters["weight"].to(x.dtype)
        # [spatial..., in, out] -> [out, in, spatial...]
        w = w.permute(nd + 1, nd, *range(nd))
        xc = x.movedim(-1, 1)
        if not xc.is_cuda:
            # The channels-last view is what cuDNN likes; the CPU kernels (oneDNN) have corrupted the
            # heap on such views with few output channels and several threads, so they get NCHW.
            xc = xc.contiguous()
        pads = self._pad()
        flat = [p for lo_hi in reversed(pads) for p in lo_hi]
        if any(flat):
            xc = F.pad(xc, flat)
        fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
        y = fn(xc, w, None, stride=tuple(cfg.strides), dilation=dil, groups=cfg.num_input_dim_groups)
        y = y.movedim(1, -1)
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        return y

    @nowrap
    def output_shape(self, *, input_shape: Sequence[Optional[int]]) -> Sequence[Optional[int]]:
        cfg = self._config
        dil = cfg.dilation or (1,) * self.ND
        spatial = []
        for n, w, s, p, d in zip(input_shape[1:-1], cfg.window, cfg.strides, self._pad(), dil):
            spatial.append(None if n is None else conv_output_length(n, window=w, stride=s, padding=p, dilation=d))
        return [input_shape[0], *spatial, cfg.output_dim]


class Conv1D(_ConvND):
    """``[B, T, C] -> [B, T', C']``; ``window`` / ``strides`` are ints."""

    ND = 1

    @config_class
    class Config(_ConvND.Config):
        window: int = 1
        strides: int = 1
        dilation: Optional[int] = None

    def __init__(self, cfg, *, parent=None):
        cfg = cfg.clone()
        super().__init__(cfg, parent=parent)

    @property
    def _tuple_cfg(self):
        return self._config

    def _create_layer_parameter_specs(self):
        cfg = self._config
        params = {"weight": ParameterSpec(
            shape=(cfg.window, cfg.input_dim // cfg.num_input_dim_groups, cfg.output_dim),
            mesh_axes=(None, None, "model"), factorization=FactorizationSpec(axes=(None, "row", "col")),
            fan_axes=FanAxes(in_axis=-2, out_axis=-1))}
        if cfg.bias:
            params["bias"] = ParameterSpec(shape=(cfg.output_dim,), mesh_axes=("model",))
        return params

    @nowrap
    def _pad(self):
        cfg = self._config
        return _explicit_padding(cfg.padding, (cfg.window,), (cfg.strides,), (cfg.dilation or 1,))

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        w = self.parameters["weight"].to(x.dtype).permute(2, 1, 0)
        xc = x.transpose(1, 2)
        (lo, hi), = self._pad()
        if lo or hi:
            xc = F.pad(xc, (lo, hi))
        y = F.conv1d(xc, w, None, stride=cfg.strides, dilation=cfg.dilation or 1, groups=cfg.num_input_dim_groups)
        y = y.transpose(1, 2)
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        return y

    @nowrap
    def output_shape(self, *, input_shape):
        cfg = self._config
        (pad,) = self._pad()
        n = input_shape[1]
        t = None if n is None else conv_output_length(n, window=cfg.window, stride=cfg.strides, padding=pad,
                                                      dilation=cfg.dilation or 1)
        return [input_shape[0], t, cfg.output_dim]


class DepthwiseConv1D(Conv1D):
    """One filter per channel (``num_input_dim_groups = input_dim``), weight ``[window, 1, dim]``."""

    @config_class
    class Config(Conv1D.Config):
        output_dim: Optional[int] = None

    def __init__(self, cfg, *, parent=None):
        cfg = cfg.clone(output_dim=cfg.input_dim, num_input_dim_groups=cfg.input_dim)
        super().__init__(cfg, parent=parent)


class Conv2D(_ConvND):
    ND = 2


class Conv3D(_ConvND):
    ND = 3

    @config_class
    class Config(_ConvND.Config):
        window: Sequence[int] = (1, 1, 1)
        strides: Sequence[int] = (1, 1, 1)


class Conv2DTranspose(BaseLayer):
    """Transposed 2-D convolution, weight ``[h, w, out, in]`` applied as the gradient of a
    ``VALID`` / ``SAME`` convolution."""

    @config_class
    class Config(BaseLayer.Config):
        window: Sequence[int] = (1, 1)
        strides: Sequence[int] = (1, 1)
        padding: str = "SAME"
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        bias: bool = True

    def _create_layer_parameter_specs(self):
        cfg = self._config
        params = {"weight": ParameterSpec(shape=tuple(cfg.window) + (cfg.output_dim, cfg.input_dim),
                                          mesh_axes=(None, None, "model", None),
                                          fan_axes=FanAxes(in_axis=-1, out_axis=-2))}
        if cfg.bias:
            params["bias"] = ParameterSpec(shape=(cfg.output_dim,), mesh_axes=("model",))
        return params

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        w = self.parameters["weight"].to(x.dtype).permute(3, 2, 0, 1)     # [in, out, h, w]
        y = F.conv_transpose2d(x.permute(0, 3, 1, 2), w, None, stride=tuple(cfg.strides))
        if cfg.padding == "SAME":
            # Crop to input * stride.
            th, tw = x.shape[1] * cfg.strides[0], x.shape[2] * cfg.strides[1]
            oh, ow = (y.shape[2] - th) // 2, (y.shape[3] - tw) // 2
            y = y[:, :, oh:oh + th, ow:ow + tw]
        y = y.permute(0, 2, 3, 1)
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        return y


class Conv2DWith1DPadding(Conv2D):
    """2-D convolution over ``[B, T, F, C]`` that also maps the ``[B, T]`` padding mask through
    the time dim (a window position is padding if its anchor frame is)."""

    def forward(self, x: Tensor, *, paddings: Tensor):  # pylint: disable=arguments-differ
        cfg = self._config
        y = super().forward(x * (1 - paddings[:, :, None, None]).to(x.dtype))
        (lo, hi) = self._pad()[0]
        p = F.pad(paddings.float(), (lo, hi), value=1.0)
        # The anchor of a window is the frame that sits where the first real frame sits in the
        # first window: `lo` frames in (0 for VALID, the centre for SAME, the last for CAUSAL).
        anchor = lo
        out_p = p[:, anchor::cfg.strides[0]][:, :y.shape[1]]
        return y * (1 - out_p[:, :, None, None]).to(y.dtype), out_p


class StackOverTime(BaseLayer):
    """``[B, T, D] -> [B, T / stride, D * stride]`` by stacking consecutive frames."""

    @config_class
    class Config(BaseLayer.Config):
        stride: Required[int] = REQUIRED

    def forward(self, x: Tensor, *, paddings: Optional[Tensor] = None):
        s = self._config.stride
        b, t, d = x.shape
        t2 = t // s
        y = x[:, :t2 * s].reshape(b, t2, s * d)
        if paddings is None:
            return y
        p = paddings[:, :t2 * s].reshape(b, t2, s).amax(dim=-1)
        return y * (1 - p[..., None]).to(y.dtype), p
