"""Causal convolutions that can be advanced chunk by chunk with an explicit cache.

Parity target: axlearn/audio/streaming/convolutions.py -- ``CausalConv2DWith1DPadding`` :27,
``CausalConv1D`` :150, ``CausalConv1DWithPadding`` :255, ``CausalConv1DTranspose`` :343.

A causal convolution with window ``w`` (dilated), stride ``s`` pads ``(w - s, s - 1)`` in time.
Streaming keeps the last ``w - s`` input frames as state: ``extend_step`` prepends them to the new
chunk (whose length must be a multiple of ``s``), convolves without left padding, and keeps the
tail as the next state -- the chunked outputs concatenate to exactly the full-sequence output.
The transposed convolution (up-sampling by ``s``) keeps ``ceil((w - 1) / s)`` input frames.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_layer import BaseLayer, FanAxes, ParameterSpec
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.convolution import Conv1D, Conv2DWith1DPadding, conv_explicit_padding
from axlearn_b200.audio.streaming.streaming_base import StreamingBase, config_method
from axlearn_b200.common.module import nowrap

Tensor = torch.Tensor


def _keep(paddings: Tensor, like: Tensor) -> Tensor:
    """1 where a frame is real, broadcast over the trailing dims of ``like``."""
    keep = (1 - paddings.to(like.dtype))
    return keep.reshape(keep.shape + (1,) * (like.dim() - keep.dim()))


def _strided_paddings(paddings: Tensor, *, stride: int, pad_left: int, pad_right: int, window: int,
                      anchor: int) -> Tensor:
    """Padding bit of every output frame: that of the input frame under its window's anchor."""
    p = F.pad(paddings.float(), (pad_left, pad_right), value=1.0)
    n_out = (p.shape[1] - window) // stride + 1
    return p[:, anchor::stride][:, :n_out]


class CausalConv1D(StreamingBase, Conv1D):
    """``[B, T, C] -> [B, T / stride, C']`` with CAUSAL padding and ``extend_step``."""

    @classmethod
    def default_config(cls):
        return super().default_config().set(padding="CAUSAL")

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.padding != "CAUSAL":
            raise ValueError(f"Only CAUSAL padding is supported (got {cfg.padding}).")

    @staticmethod
    def _cfg_time_padding(cfg) -> tuple:
        return tuple(conv_explicit_padding("CAUSAL", (cfg.window,), (cfg.strides,), (cfg.dilation or 1,))[0])

    @nowrap
    def _time_padding(self) -> tuple:
        return self._cfg_time_padding(self._config)

    @nowrap
    def cache_size(self) -> int:
        return self._time_padding()[0]

    @config_method
    def in_stride(cls, cfg) -> int:  # pylint: disable=no-self-argument
        return cfg.strides

    @config_method
    def segment_pad(cls, cfg) -> int:  # pylint: disable=no-self-argument
        """Padding frames needed between packed segments so that no window spans two of them."""
        return max(cls._cfg_time_padding(cfg))

    @nowrap
    def init_states(self, *, batch_size: int, dtype: torch.dtype = torch.float32, device=None) -> dict:
        cfg = self._config
        return {"x": torch.zeros(batch_size, self.cache_size(), cfg.input_dim, dtype=dtype, device=device)}

    def _conv_no_left_pad(self, context: Tensor) -> Tensor:
        cfg = self._config
        w = self.parameters["weight"].to(context.dtype).permute(2, 1, 0)
        xc = context.transpose(1, 2)
        hi = self._time_padding()[1]
        if hi:
            xc = F.pad(xc, (0, hi))
        y = F.conv1d(xc, w, None, stride=cfg.strides, dilation=cfg.dilation or 1, groups=cfg.num_input_dim_groups)
        y = y.transpose(1, 2)
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        return y

    def extend_step(self, *, cached_states: dict, input_data: dict, is_prefill: bool = False):
        """``input_data["x"] [B, T, C]`` with ``T % stride == 0`` -> ``(states, {"x": [B, T / stride, C']})``."""
        del is_prefill
        cfg = self._config
        x = input_data["x"]
        if x.shape[1] % cfg.strides:
            raise ValueError(f"The number of time steps {x.shape[1]} must be divisible by the stride {cfg.strides}.")
        context = torch.cat([cached_states["x"].to(x.dtype), x], dim=1)
        y = self._conv_no_left_pad(context)[:, : x.shape[1] // cfg.strides]
        cache = self.cache_size()
        states = dict(cached_states, x=context[:, context.shape[1] - cache:] if cache > 0 else cached_states["x"])
        return states, {"x": y}


class CausalConv1DWithPadding(CausalConv1D):
    """The same with a ``[B, T]`` padding mask: padded frames are zeroed on the way in and out, and
    the mask is carried through the stride (an output frame is padding if the LAST input frame of
    its stride group is)."""

    def forward(self, x: Tensor, *, paddings: Tensor):  # pylint: disable=arguments-differ
        y = super().forward(x * _keep(paddings, x))
        out_p = self.conv_paddings(paddings)
        return y * _keep(out_p, y), out_p

    @nowrap
    def conv_paddings(self, paddings: Tensor) -> Tensor:
        cfg = self._config
        lo, hi = self._time_padding()
        eff = (cfg.window - 1) * (cfg.dilation or 1) + 1
        return _strided_paddings(paddings, stride=cfg.strides, pad_left=lo, pad_right=hi, window=eff, anchor=eff - 1)

    @nowrap
    def init_states(self, *, batch_size: int, dtype: torch.dtype = torch.float32, device=None) -> dict:
        states = super().init_states(batch_size=batch_size, dtype=dtype, device=device)
        states["paddings"] = torch.zeros(batch_size, self.cache_size(), dtype=torch.bool, device=device)
        return states

    def extend_step(self, *, cached_states: dict, input_data: dict, is_prefill: bool = False):
        x, paddings = input_data["x"], input_data["paddings"]
        states, out = super().extend_step(cached_states=cached_states,
                                          input_data={"x": x * _keep(paddings, x)}, is_prefill=is_prefill)
        # Within a chunk the anchor of output j is input frame (j + 1) * stride - 1.
        s = self._config.strides
        out_p = paddings[:, s - 1::s]
        cache = self.cache_size()
        ctx_p = torch.cat([cached_states["paddings"], paddings.bool()], dim=1)
        states["paddings"] = ctx_p[:, ctx_p.shape[1] - cache:] if cache > 0 else cached_states["paddings"]
        return states, {"x": out["x"] * _keep(out_p, out["x"]), "paddings": out_p}


class CausalConv2DWith1DPadding(StreamingBase, Conv2DWith1DPadding):
    """``[B, T, F, C]`` convolution, causal in time (SAME in frequency), with ``extend_step``."""

    @classmethod
    def default_config(cls):
        return super().default_config().set(padding="CAUSAL")

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.padding != "CAUSAL":
            raise ValueError(f"Only CAUSAL padding is supported (got {cfg.padding}).")

    @nowrap
    def _time_padding(self) -> tuple:
        return tuple(self._pad()[0])

    @nowrap
    def cache_size(self) -> int:
        return self._time_padding()[0]

    @config_method
    def in_stride(cls, cfg) -> int:  # pylint: disable=no-self-argument
        return cfg.strides[0]

    @config_method
    def segment_pad(cls, cfg) -> int:  # pylint: disable=no-self-argument
        dil = cfg.dilation or (1,) * len(cfg.window)
        return max(conv_explicit_padding(cfg.padding, cfg.window, cfg.strides, dil)[0])

    def forward(self, x: Tensor, *, paddings: Tensor):
        cfg = self._config
        y = super(Conv2DWith1DPadding, self).forward(x * _keep(paddings, x))
        out_p = self.conv_paddings(paddings)
        return y * _keep(out_p, y), out_p

    @nowrap
    def conv_paddings(self, paddings: Tensor) -> Tensor:
        cfg = self._config
        lo, hi = self._time_padding()
        eff = (cfg.window[0] - 1) * ((cfg.dilation or (1, 1))[0]) + 1
        return _strided_paddings(paddings, stride=cfg.strides[0], pad_left=lo, pad_right=hi, window=eff, anchor=eff - 1)

    @nowrap
    def init_states(self, *, batch_size: int, feature_dim: int, dtype: torch.dtype = torch.float32, device=None) -> dict:
        cfg = self._config
        cache = self.cache_size()
        return {"x": torch.zeros(batch_size, cache, feature_dim, cfg.input_dim, dtype=dtype, device=device),
                "paddings": torch.zeros(batch_size, cache, dtype=torch.bool, device=device)}

    def extend_step(self, *, cached_states: dict, input_data: dict, is_prefill: bool = False):
        del is_prefill
        cfg = self._config
        stride = cfg.strides[0]
        x, paddings = input_data["x"], input_data["paddings"]
        if x.shape[1] % stride:
            raise ValueError(f"The number of time steps {x.shape[1]} must be divisible by the stride {stride}.")
        x = x * _keep(paddings, x)
        context = torch.cat([cached_states["x"].to(x.dtype), x], dim=1)
        ctx_p = torch.cat([cached_states["paddings"], paddings.bool()], dim=1)
        context = context * _keep(ctx_p, context)
        # Past context is explicit: no left padding in time; the other dims keep theirs.
        pads = self._pad()
        step_pads = [(0, pads[0][1])] + [tuple(p) for p in pads[1:]]
        nd = 2
        dil = tuple(cfg.dilation or (1,) * nd)
        w = self.parameters["weight"].to(x.dtype).permute(nd + 1, nd, *range(nd))
        xc = context.movedim(-1, 1).contiguous()
        flat = [p for lo_hi in reversed(step_pads) for p in lo_hi]
        if any(flat):
            xc = F.pad(xc, flat)
        y = F.conv2d(xc, w, None, stride=tuple(cfg.strides), dilation=dil, groups=cfg.num_input_dim_groups).movedim(1, -1)
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        y = y[:, : x.shape[1] // stride]
        out_p = paddings[:, stride - 1::stride]
        cache = self.cache_size()
        states = {"x": context[:, context.shape[1] - cache:] if cache > 0 else cached_states["x"],
                  "paddings": ctx_p[:, ctx_p.shape[1] - cache:] if cache > 0 else cached_states["paddings"]}
        return states, {"x": y * _keep(out_p, y), "paddings": out_p}


class Conv1DTranspose(BaseLayer):
    """Transposed 1-D convolution ``[B, T, C] -> [B, T * stride (+ edge), C']``, weight
    ``[window, in, out]`` (axlearn/common/convolution.py ``Conv1DTranspose``).  Padding names are
    those of the forward convolution whose transpose this is: SAME -> ``T * stride`` outputs
    centred, VALID -> ``T * stride + max(window - stride, 0)``, CAUSAL -> ``T * stride`` outputs
    that depend on past and present inputs only."""

    @config_class
    class Config(BaseLayer.Config):
        window: int = 1
        strides: int = 1
        padding: str = "SAME"
        dilation: int = 1
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        bias: bool = True

    def _create_layer_parameter_specs(self):
        cfg = self._config
        params = {"weight": ParameterSpec(shape=(cfg.window, cfg.input_dim, cfg.output_dim),
                                          mesh_axes=(None, None, "model"), fan_axes=FanAxes(in_axis=-2, out_axis=-1))}
        if cfg.bias:
            params["bias"] = ParameterSpec(shape=(cfg.output_dim,), mesh_axes=("model",))
        return params

    @nowrap
    def _full_and_crop(self, t: int) -> tuple:
        """``(length of the uncropped result, first kept index, kept length)``."""
        cfg = self._config
        eff = (cfg.window - 1) * cfg.dilation + 1
        full = (t - 1) * cfg.strides + eff
        if cfg.padding == "VALID":
            return full, 0, t * cfg.strides + max(eff - cfg.strides, 0)
        if cfg.padding == "CAUSAL":
            return full, 0, t * cfg.strides
        if cfg.padding == "SAME":
            extra = max(eff - cfg.strides, 0)
            return full, extra // 2, t * cfg.strides
        raise NotImplementedError(cfg.padding)

    def _raw(self, x: Tensor) -> Tensor:
        cfg = self._config
        w = self.parameters["weight"].to(x.dtype).permute(1, 2, 0)      # [in, out, window]
        return F.conv_transpose1d(x.transpose(1, 2), w, None, stride=cfg.strides, dilation=cfg.dilation).transpose(1, 2)

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        full, lo, n = self._full_and_crop(x.shape[1])
        y = self._raw(x)
        if n > full:
            y = F.pad(y, (0, 0, 0, n - full))
        y = y[:, lo: lo + n]
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        return y

    @nowrap
    def output_shape(self, *, input_shape):
        _, _, n = self._full_and_crop(input_shape[1])
        return [input_shape[0], n, self._config.output_dim]


class CausalConv1DTranspose(StreamingBase, Conv1DTranspose):
    """Causal up-sampling with ``extend_step``: output frames ``[t * s, (t + 1) * s)`` depend on
    inputs ``t, t - 1, ..., t - ceil((w - 1) / s)``; the state holds those past input frames."""

    @classmethod
    def default_config(cls):
        return super().default_config().set(padding="CAUSAL")

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.padding != "CAUSAL":
            raise ValueError(f"Only CAUSAL padding is supported (got {cfg.padding}).")

    @nowrap
    def cache_size(self) -> int:
        cfg = self._config
        eff = (cfg.window - 1) * cfg.dilation + 1
        return math.ceil((eff - 1) / cfg.strides)

    @config_method
    def out_stride(cls, cfg) -> int:  # pylint: disable=no-self-argument
        return cfg.strides

    @config_method
    def segment_pad(cls, cfg) -> int:  # pylint: disable=no-self-argument
        # Output frame o sees input frames t with t * s <= o <= t * s + (w - 1) * d; the zeros that
        # up-sampling puts between inputs count as padding, so floor, not ceil.
        return max((cfg.window - 1) * cfg.dilation, cfg.strides - 1) // cfg.strides

    @nowrap
    def init_states(self, *, batch_size: int, dtype: torch.dtype = torch.float32, device=None) -> dict:
        cfg = self._config
        cache = self.cache_size()
        return {"x": torch.zeros(batch_size, cache, cfg.input_dim, dtype=dtype, device=device),
                "paddings": torch.ones(batch_size, cache, dtype=torch.bool, device=device)}

    def extend_step(self, *, cached_states: dict, input_data: dict, is_prefill: bool = False):
        del is_prefill
        cfg = self._config
        x = input_data["x"]
        cache = self.cache_size()
        context = torch.cat([cached_states["x"].to(x.dtype), x], dim=1)
        states = dict(cached_states)
        if "paddings" in input_data:
            ctx_p = torch.cat([cached_states["paddings"], input_data["paddings"].bool()], dim=1)
            context = context * _keep(ctx_p, context)
            states["paddings"] = ctx_p[:, ctx_p.shape[1] - cache:] if cache > 0 else cached_states["paddings"]
        # Outputs of the new frames start `cache * stride` frames into the raw result of the context.
        raw = self._raw(context)
        start = cache * cfg.strides
        y = raw[:, start: start + x.shape[1] * cfg.strides]
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        states["x"] = context[:, context.shape[1] - cache:] if cache > 0 else cached_states["x"]
        out = {"x": y}
        if "paddings" in input_data:
            out_p = input_data["paddings"].repeat_interleave(cfg.strides, dim=1)
            out = {"x": y * _keep(out_p, y), "paddings": out_p}
        return states, out
