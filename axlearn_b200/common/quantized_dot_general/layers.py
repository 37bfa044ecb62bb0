"""Quantised contractions for dense layers.

Parity target in the reference: ``QuantizedDotGeneral`` (axlearn/common/quantized_dot_general/
layers.py:69-203, 282-323; fp8_ops.py:15-257): a child layer that dense layers call instead of a
plain einsum, configured by ``quantization_type`` (fp8 / int8) and, for fp8,
``fp8_amax_history_length``.

Two fp8 schemes:

* ``scaling="tensor"``: the reference's per-tensor scaling.  Every dense layer owns six extra
  parameters -- ``input_scale``, ``kernel_scale``, ``output_grad_scale`` (fp32 scalars, initial
  1) and, with a history length > 0 (*delayed* scaling), ``input_amax_history``,
  ``kernel_amax_history``, ``output_grad_amax_history`` (``[length]``, initial 0).  A forward pass
  quantises with the scale derived from the *stored* history, and the new scales / histories
  come back from ``backward`` **as the gradients of those parameters**; the learner applies
  them as in-place overrides (``OverrideInplaceUpdateTransformation`` with rules
  ``.*/<name>``, installed by ``FP8ConfigModifier``), so they are part of the checkpointed
  state under the reference's names.  With history length 0 / None the scale comes from the
  current tensor (in-batch scaling) and only the three scale parameters exist.
* ``scaling="block"`` (default here): 1x128 activation / 128x128 weight scale blocks computed
  from the current tensors (``ops/fp8_ops.py``) -- no state, and the form the tcgen05 fp8 kernel
  runs.
"""

from __future__ import annotations

import enum
from typing import Optional

import torch

from axlearn_b200 import ops
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common import prng
from axlearn_b200.common.config import InstantiableConfig, config_class
from axlearn_b200.common.param_init import constant_initializer
from axlearn_b200.ops import fp8_ops

Tensor = torch.Tensor

FP8_SCALE_PARAMS = ("input_scale", "kernel_scale", "output_grad_scale")
FP8_AMAX_HISTORY_PARAMS = ("input_amax_history", "kernel_amax_history", "output_grad_amax_history")


def get_all_fp8_param_names() -> list[str]:
    return list(FP8_SCALE_PARAMS) + list(FP8_AMAX_HISTORY_PARAMS)


class DotGeneralQuantizationType(enum.Enum):
    INT_8 = "int8"
    FP_8 = "fp8"


class ClippingChoice(enum.Enum):
    """Which tensor the activation-clipping child is applied to."""

    INPUT_ACTIVATION = 0
    OUTPUT_ACTIVATION = 1


def compute_scale(amax: Tensor, scale: Tensor, fp8_max: float) -> Tensor:
    """New dequantisation scale from an amax (reference math: flax ``fp8_ops.compute_scale`` with
    margin 0): ``amax / fp8_max`` where amax is positive and finite, else the old scale."""
    ok = torch.isfinite(amax) & (amax > 0)
    return torch.where(ok, amax / fp8_max, scale)


def update_amax_history(x: Tensor, history: Tensor) -> Tensor:
    """Rolls the history by one and stores ``max|x|`` in slot 0."""
    new = torch.roll(history, shifts=-1, dims=0).clone()
    new[0] = x.detach().abs().amax().to(history.dtype)
    return new


def _quantize(x: Tensor, scale: Tensor, history: Optional[Tensor], *, e5m2: bool):
    """``(dequantised fp8 value of x, new_scale, new_history)``; delayed scaling when ``history``
    is given (the scale comes from the stored history, which then takes the current amax)."""
    fmax = fp8_ops.E5M2_MAX if e5m2 else fp8_ops.E4M3_MAX
    if history is None:
        amax, new_history = x.detach().abs().amax().float(), None
    else:
        amax, new_history = history.max(), update_amax_history(x, history)
    new_scale = compute_scale(amax, scale.float(), fmax)
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    q = (x.float() / new_scale).clamp(-fmax, fmax).to(dt)
    return q.float() * new_scale, new_scale.to(scale.dtype), new_history


class _TensorScaledFp8(torch.autograd.Function):
    """Per-tensor scaled fp8 matmul: e4m3 forward operands, e5m2 output gradient, fp32
    accumulation.  The gradients returned for the scale / history inputs are their NEW VALUES."""

    @staticmethod
    def forward(ctx, x, w, in_scale, k_scale, og_scale, in_hist, k_hist, og_hist):
        xq, new_in_scale, new_in_hist = _quantize(x, in_scale, in_hist, e5m2=False)
        wq, new_k_scale, new_k_hist = _quantize(w, k_scale, k_hist, e5m2=False)
        ctx.save_for_backward(xq, wq, og_scale, og_hist if og_hist is not None else og_scale.new_zeros(0))
        ctx.has_hist = og_hist is not None
        ctx.new = (new_in_scale, new_k_scale, new_in_hist, new_k_hist)
        ctx.dtypes = (x.dtype, w.dtype)
        return (xq @ wq).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        xq, wq, og_scale, og_hist = ctx.saved_tensors
        dyq, new_og_scale, new_og_hist = _quantize(dy, og_scale, og_hist if ctx.has_hist else None, e5m2=True)
        new_in_scale, new_k_scale, new_in_hist, new_k_hist = ctx.new
        dx = (dyq @ wq.t()).to(ctx.dtypes[0]) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = (xq.reshape(-1, xq.shape[-1]).t() @ dyq.reshape(-1, dy.shape[-1])).to(ctx.dtypes[1])
        return dx, dw, new_in_scale, new_k_scale, new_og_scale, new_in_hist, new_k_hist, new_og_hist


class QuantizedDotGeneral(BaseLayer):
    """``matmul(x [..., K], w [K, N])`` in reduced precision."""

    @config_class
    class Config(BaseLayer.Config):
        quantization_type: Optional[DotGeneralQuantizationType] = DotGeneralQuantizationType.FP_8
        fp8_amax_history_length: int = 128
        scaling: str = "block"   # "block" | "tensor"
        # int8 only: a BaseActivationClippingLayer config applied to the input or the output.
        activation_clipping: Optional[InstantiableConfig] = None
        clipping_choice: ClippingChoice = ClippingChoice.INPUT_ACTIVATION

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if self._config.activation_clipping is not None:
            self._add_child("activation_clipping", self._config.activation_clipping)

    def _create_layer_parameter_specs(self):
        cfg = self._config
        if cfg.quantization_type != DotGeneralQuantizationType.FP_8 or cfg.scaling != "tensor":
            return {}
        scale = lambda: ParameterSpec(shape=(), dtype=torch.float32, mesh_axes=(),
                                      initializer=constant_initializer(1.0), weight_decay_scale=0.0)
        specs = {name: scale() for name in FP8_SCALE_PARAMS}
        if cfg.fp8_amax_history_length and cfg.fp8_amax_history_length > 0:
            hist = lambda: ParameterSpec(shape=(cfg.fp8_amax_history_length,), dtype=torch.float32,
                                         mesh_axes=(None,), initializer=constant_initializer(0.0),
                                         weight_decay_scale=0.0)
            specs.update({name: hist() for name in FP8_AMAX_HISTORY_PARAMS})
        return specs

    def matmul(self, x: Tensor, w: Tensor) -> Tensor:
        cfg = self._config
        if cfg.quantization_type is None:
            return ops.linear(x, w)
        if cfg.quantization_type == DotGeneralQuantizationType.INT_8:
            clip = self._children.get("activation_clipping")
            if clip is not None and cfg.clipping_choice == ClippingChoice.INPUT_ACTIVATION:
                x = clip(x)
            # Stochastic rounding of the output gradient draws from this layer's PRNG stream
            # while training (deterministic round-to-nearest otherwise).
            seed = None
            key = self.get_invocation_context().prng_key
            if self.is_training and key is not None:
                seed = prng.seed_of(key) % (2**31 - 1)
            y = _Int8DotGeneral.apply(x, w.to(x.dtype), seed)
            if clip is not None and cfg.clipping_choice == ClippingChoice.OUTPUT_ACTIVATION:
                y = clip(y)
            return y
        if cfg.scaling == "tensor":
            params = self.parameters
            delayed = "input_amax_history" in params
            # The trainer's bf16 working copies of these fp32 parameters would lose the scales'
            # precision: they are read (and their new values returned) in fp32.
            f32 = lambda name: params[name] if params[name].dtype == torch.float32 else params[name].float()
            scales = [f32(n) for n in FP8_SCALE_PARAMS]
            hists = [f32(n) for n in FP8_AMAX_HISTORY_PARAMS] if delayed else [None, None, None]
            return _TensorScaledFp8.apply(x, w.to(x.dtype), *scales, *hists)
        if cfg.scaling != "block":
            raise NotImplementedError(cfg.scaling)
        w = w.to(x.dtype)
        if not fp8_ops.supported(x, w):
            return ops.linear(x, w)     # odd shapes (tiny heads, ragged token counts) stay in bf16
        return fp8_ops.fp8_linear(x, w)


def _quantize_int8(t: Tensor, dim: int, *, noise: Optional[Tensor] = None) -> tuple[Tensor, Tensor]:
    """Symmetric int8 along ``dim`` (the contraction dim): returns the integer-valued tensor (in
    ``t``'s dtype; every integer in [-127, 127] is exact in bf16) and the fp32 scales.  With
    ``noise`` (uniform in [0, 1)) the rounding is stochastic: ``floor(v + u)``, unbiased."""
    scale = t.detach().abs().amax(dim=dim, keepdim=True).float().clamp_min(1e-30) / 127.0
    v = t.float() / scale
    q = torch.floor(v + noise) if noise is not None else torch.round(v)
    return q.clamp(-127, 127).to(t.dtype), scale


class _Int8DotGeneral(torch.autograd.Function):
    """``x [..., K] @ w [K, N]`` on the int8 grid, the reference's default recipe (AQT ``config_v3``
    through ``lhs_activation_aqt_config``, axlearn/common/quantized_dot_general/utils.py:26-48):

    * forward: activations quantised per row, weights per output column (both over K), products
      accumulated exactly, result rescaled by the two scales;
    * input gradient: the output gradient quantised per row over N with STOCHASTIC rounding and
      the weights re-quantised per input row (over N);
    * weight gradient: not quantised.

    The integer-valued operands travel as bf16 (exact) through the framework's tensor-core GEMM
    with fp32 accumulation; an int32 accumulator would differ only where a sum exceeds 2^24."""

    @staticmethod
    def forward(ctx, x, w, seed):
        xq, sx = _quantize_int8(x, -1)
        wq, sw = _quantize_int8(w, 0)
        ctx.save_for_backward(x, w)
        ctx.seed = seed
        y = ops.linear(xq, wq).float() * sx * sw
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = dw = None
        if ctx.needs_input_grad[0]:
            noise = None
            if ctx.seed is not None:
                gen = torch.Generator(device=dy.device).manual_seed(ctx.seed)
                noise = torch.rand(dy.shape, generator=gen, device=dy.device, dtype=torch.float32)
            gq, sg = _quantize_int8(dy, -1, noise=noise)
            wq, sw = _quantize_int8(w, 1)                                  # per input row, over N
            dx = (ops.linear(gq, wq.t().contiguous()).float() * sg * sw.reshape(-1)).to(x.dtype)
        if ctx.needs_input_grad[1]:
            dw = (x.reshape(-1, x.shape[-1]).t().float() @ dy.reshape(-1, dy.shape[-1]).float()).to(w.dtype)
        return dx, dw, None
