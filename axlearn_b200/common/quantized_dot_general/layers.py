"""Quantised contractions for dense layers.

Parity target in the reference: ``QuantizedDotGeneral`` (axlearn/common/quantized_dot_general/
layers.py): a child layer that dense layers call instead of a plain einsum, configured by
``quantization_type`` (fp8 / int8) and, for fp8, ``fp8_amax_history_length``.  The reference
quantises per tensor with delayed scaling (scales from a history of amax values kept as
parameters whose "gradients" overwrite them in place).

Two fp8 schemes are offered here:

* ``scaling="block"`` (default): 1x128 activation / 128x128 weight scale blocks computed from the
  current tensors (``ops/fp8_ops.py``) -- no state, and the form the tcgen05 kernel runs;
* ``scaling="tensor"``: one scale per tensor from the current amax, with the amax histories kept
  as state (``*_amax_history`` parameters updated through state updates) for parity of the
  parameter tree and for monitoring.
"""

from __future__ import annotations

import enum
from typing import Optional

import torch

from axlearn_b200 import ops
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import config_class
from axlearn_b200.common.module import nowrap
from axlearn_b200.common.param_init import constant_initializer
from axlearn_b200.ops import fp8_ops

Tensor = torch.Tensor


class DotGeneralQuantizationType(enum.Enum):
    INT_8 = "int8"
    FP_8 = "fp8"


class _TensorScaledFp8(torch.autograd.Function):
    """Per-tensor current scaling: e4m3 forward operands, e5m2 gradients, fp32 accumulation."""

    @staticmethod
    def forward(ctx, x, w):
        def q(t, e5m2=False):
            amax = t.detach().abs().amax().float().clamp_min(1e-12)
            s = amax / (fp8_ops.E5M2_MAX if e5m2 else fp8_ops.E4M3_MAX)
            return (t.float() / s).to(torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn).float() * s

        ctx.q = q
        ctx.save_for_backward(x, w)
        return (q(x) @ q(w)).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        q = ctx.q
        dyq = q(dy, e5m2=True)
        dx = (dyq @ q(w).t()).to(x.dtype) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            x2 = q(x).reshape(-1, x.shape[-1])
            dw = (x2.t() @ dyq.reshape(-1, dy.shape[-1])).to(w.dtype)
        return dx, dw


class QuantizedDotGeneral(BaseLayer):
    """``matmul(x [..., K], w [K, N])`` in reduced precision."""

    @config_class
    class Config(BaseLayer.Config):
        quantization_type: Optional[DotGeneralQuantizationType] = DotGeneralQuantizationType.FP_8
        fp8_amax_history_length: int = 128
        scaling: str = "block"   # "block" | "tensor"

    def _create_layer_parameter_specs(self):
        cfg = self._config
        if cfg.quantization_type != DotGeneralQuantizationType.FP_8 or cfg.scaling != "tensor":
            return {}
        hist = lambda: ParameterSpec(shape=(cfg.fp8_amax_history_length,), dtype=torch.float32, mesh_axes=(None,),
                                     initializer=constant_initializer(0.0), weight_decay_scale=0.0)
        return {"input_amax_history": hist(), "kernel_amax_history": hist(), "output_grad_amax_history": hist()}

    @nowrap
    def _record_amax(self, name: str, t: Tensor) -> None:
        hist = self.parameters[name].detach()
        new = torch.roll(hist, 1)
        new[0] = t.detach().abs().amax().float()
        self.add_state_update(name, new)

    def matmul(self, x: Tensor, w: Tensor) -> Tensor:
        cfg = self._config
        if cfg.quantization_type is None:
            return ops.linear(x, w)
        if cfg.quantization_type == DotGeneralQuantizationType.INT_8:
            return _int8_matmul(x, w)
        if cfg.scaling == "tensor":
            self._record_amax("input_amax_history", x)
            self._record_amax("kernel_amax_history", w)
            return _TensorScaledFp8.apply(x, w.to(x.dtype))
        if cfg.scaling != "block":
            raise NotImplementedError(cfg.scaling)
        w = w.to(x.dtype)
        if not fp8_ops.supported(x, w):
            return ops.linear(x, w)     # odd shapes (tiny heads, ragged token counts) stay in bf16
        return fp8_ops.fp8_linear(x, w)


def _int8_matmul(x: Tensor, w: Tensor) -> Tensor:
    """Symmetric per-row (activations) / per-column (weights) int8 with a straight-through
    gradient."""
    sx = x.detach().abs().amax(dim=-1, keepdim=True).float().clamp_min(1e-12) / 127.0
    sw = w.detach().abs().amax(dim=0, keepdim=True).float().clamp_min(1e-12) / 127.0
    xq = torch.round(x.float() / sx).clamp(-127, 127) * sx
    wq = torch.round(w.float() / sw).clamp(-127, 127) * sw
    # Straight-through: forward uses the quantised values, backward the identity.
    xs = x.float() + (xq - x.float()).detach()
    ws = w.float() + (wq - w.float()).detach()
    return (xs @ ws).to(x.dtype)
