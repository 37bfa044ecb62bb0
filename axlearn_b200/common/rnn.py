"""Recurrent layers.

Parity targets in the reference (axlearn/common/rnn.py): ``BaseRNNCell`` with
``init_states(batch_size)`` / ``extend_step(cached_states, data)`` / ``forward(time_major_inputs)``,
``LSTMCell`` (one fused ``[input_dim + hidden_dim, 4 * hidden_dim]`` projection, optional output
projection and cell-value clipping), ``StackedRNNLayer`` and ``IdentityCell``.
Inputs to ``forward`` are time-major ``[T, B, D]`` like the reference's.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Linear

Tensor = torch.Tensor


class BaseRNNCell(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Optional[int] = None

    def init_states(self, *, batch_size: int, device=None):
        raise NotImplementedError(type(self))

    def extend_step(self, *, cached_states, data: Tensor):
        raise NotImplementedError(type(self))

    def forward(self, time_major_inputs: Tensor) -> Tensor:
        states = self.init_states(batch_size=time_major_inputs.shape[1], device=time_major_inputs.device)
        outs = []
        for t in range(time_major_inputs.shape[0]):
            states, y = self.extend_step(cached_states=states, data=time_major_inputs[t])
            outs.append(y)
        return torch.stack(outs, dim=0)


class IdentityCell(BaseRNNCell):
    def init_states(self, *, batch_size, device=None):
        return {}

    def extend_step(self, *, cached_states, data):
        return cached_states, data


class LSTMCell(BaseRNNCell):
    @config_class
    class Config(BaseRNNCell.Config):
        hidden_dim: Optional[int] = None
        max_cell_value: Optional[float] = None
        output_proj: Optional[InstantiableConfig] = None
        input_proj: InstantiableConfig = Linear.default_config().set(bias=True)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._hidden = cfg.hidden_dim or cfg.output_dim or cfg.input_dim
        self._out = cfg.output_dim or self._hidden
        self._add_child("input_proj", cfg.input_proj.clone(
            input_dim=cfg.input_dim + self._out, output_dim=4 * self._hidden, param_partition_spec=(None, None)))
        if cfg.output_proj is not None or self._out != self._hidden:
            proj = (cfg.output_proj or Linear.default_config().set(bias=False)).clone(
                input_dim=self._hidden, output_dim=self._out, param_partition_spec=(None, None))
            self._add_child("output_proj", proj)

    def init_states(self, *, batch_size, device=None):
        z = lambda d: torch.zeros(batch_size, d, device=device)
        return {"m": z(self._out), "c": z(self._hidden)}

    def extend_step(self, *, cached_states, data):
        cfg = self._config
        proj = self.input_proj(torch.cat([data, cached_states["m"].to(data.dtype)], dim=-1))
        i, f, g, o = proj.chunk(4, dim=-1)
        c = torch.sigmoid(f) * cached_states["c"].to(data.dtype) + torch.sigmoid(i) * torch.tanh(g)
        if cfg.max_cell_value is not None:
            c = c.clamp(-cfg.max_cell_value, cfg.max_cell_value)
        m = torch.sigmoid(o) * torch.tanh(c)
        if "output_proj" in self._children:
            m = self.output_proj(m)
        return {"m": m, "c": c}, m


class StackedRNNLayer(BaseRNNCell):
    """Cells applied in sequence; ``layers`` are cell configs (their dims are chained)."""

    @config_class
    class Config(BaseRNNCell.Config):
        layers: Required[Sequence[InstantiableConfig]] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        dim = cfg.input_dim
        self._cells = []
        for i, c in enumerate(cfg.layers):
            cell = self._add_child(f"layer{i}", c.clone(input_dim=dim))
            dim = c.output_dim or getattr(c, "hidden_dim", None) or dim
            self._cells.append(cell)

    def init_states(self, *, batch_size, device=None):
        return [c.init_states(batch_size=batch_size, device=device) for c in self._cells]

    def extend_step(self, *, cached_states, data):
        new = []
        for cell, st in zip(self._cells, cached_states):
            st, data = cell.extend_step(cached_states=st, data=data)
            new.append(st)
        return new, data
