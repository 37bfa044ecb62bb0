"""int8 contraction: grid values, straight gradients, stochastic rounding, clipping layers
(reference: axlearn/common/quantized_dot_general/{layers,utils,activation_clipping}.py)."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.common.quantized_dot_general.activation_clipping import (
    DummyActivationClippingLayer,
    HardActivationClippingLayer,
    TanhActivationClippingLayer,
)
from axlearn_b200.common.quantized_dot_general.layers import (
    ClippingChoice,
    DotGeneralQuantizationType,
    QuantizedDotGeneral,
    _quantize_int8,
)


def _layer(**kw):
    return QuantizedDotGeneral.default_config().set(
        name="q", quantization_type=DotGeneralQuantizationType.INT_8, **kw).instantiate(parent=None)


def test_quantiser_grid_and_stochastic_rounding_is_unbiased():
    torch.manual_seed(0)
    t = torch.randn(64, 256)
    q, s = _quantize_int8(t, -1)
    assert torch.equal(q, q.round()) and q.abs().max() <= 127
    assert ((q * s) - t).abs().max() <= 0.5 * s.max() + 1e-6       # round to nearest: half a level
    assert (q.abs().amax(dim=-1) == 127).all()                       # every row uses the full range
    # Stochastic rounding: the mean over many draws converges to the value itself.
    acc = torch.zeros_like(t)
    n = 400
    for i in range(n):
        noise = torch.rand(t.shape, generator=torch.Generator().manual_seed(i))
        qs, ss = _quantize_int8(t, -1, noise=noise)
        assert torch.equal(qs, qs.round())
        acc += qs * ss
    bias = (acc / n - t).abs().max()
    assert bias < 0.12 * s.max(), (bias, s.max())                    # << half a level (0.5 * s)


def test_forward_and_gradients_against_fp32():
    torch.manual_seed(1)
    x = torch.randn(4, 24, 64, requires_grad=True)
    w = (torch.randn(64, 48) / 8).requires_grad_()
    layer = _layer()
    y, _ = functional(layer, prng.PRNGKey(3), {}, [x, w], is_training=True, method="matmul")
    ref = x @ w
    assert (y - ref).abs().max() < 0.03 * ref.abs().max()
    g = torch.randn_like(ref)
    y.backward(g)
    dx_ref, dw_ref = g @ w.t(), x.reshape(-1, 64).t() @ g.reshape(-1, 48)
    assert (x.grad - dx_ref.detach()).abs().max() < 0.05 * dx_ref.abs().max()
    torch.testing.assert_close(w.grad, dw_ref.detach(), rtol=1e-4, atol=1e-4)   # the weight gradient is not quantised


def test_training_rounding_follows_the_prng_key_and_eval_is_deterministic():
    torch.manual_seed(2)
    x = torch.randn(8, 32)
    w = torch.randn(32, 16)
    g = torch.randn(8, 16)
    layer = _layer()

    def dx(key, training):
        xi = x.clone().requires_grad_()
        y, _ = functional(layer, key, {}, [xi, w], is_training=training, method="matmul")
        y.backward(g)
        return xi.grad

    a, b, c = dx(prng.PRNGKey(1), True), dx(prng.PRNGKey(1), True), dx(prng.PRNGKey(2), True)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert torch.equal(dx(prng.PRNGKey(1), False), dx(prng.PRNGKey(2), False))


@pytest.mark.parametrize("cls,expect", [
    (HardActivationClippingLayer, lambda x, b: x.clamp(-b, b)),
    (TanhActivationClippingLayer, lambda x, b: torch.tanh(x / b) * b),
    (DummyActivationClippingLayer, lambda x, b: x),
])
def test_clipping_layers(cls, expect):
    x = torch.tensor([-5.0, -1.0, 0.25, 2.0, 7.0])
    layer = cls.default_config().set(name="clip", clipping_max_abs=2.0, clipping_summary=True).instantiate(parent=None)
    y, col = functional(layer, None, {}, [x], is_training=True)
    torch.testing.assert_close(y, expect(x, 2.0))
    assert abs(float(col.summaries["activations/clipped_activation"]) - 0.4) < 1e-6
    with pytest.raises(ValueError):
        cls.default_config().set(name="clip", clipping_max_abs=0.0).instantiate(parent=None)


def test_clipping_inside_the_contraction_tames_an_outlier():
    torch.manual_seed(3)
    x = torch.randn(16, 64)
    x[0, 0] = 500.0                                                  # one outlier makes row 0 coarse
    w = torch.randn(64, 8) / 8
    clip = HardActivationClippingLayer.default_config().set(clipping_max_abs=4.0)
    plain = _layer()
    clipped = _layer(activation_clipping=clip, clipping_choice=ClippingChoice.INPUT_ACTIVATION)
    y0, _ = functional(plain, None, {}, [x, w], is_training=False, method="matmul")
    y1, _ = functional(clipped, None, {}, [x, w], is_training=False, method="matmul")
    ref = x.clamp(-4, 4) @ w
    assert (y1 - ref).abs().max() < 0.03 * ref.abs().max()
    rest = (x[0, 1:] @ w[1:])                                        # what row 0 carries besides the outlier
    assert ((y0[0] - x[0, 0] * w[0]) - rest).abs().max() > 5 * (y1[0] - ref[0]).abs().max()
    out = _layer(activation_clipping=HardActivationClippingLayer.default_config().set(clipping_max_abs=0.5),
                 clipping_choice=ClippingChoice.OUTPUT_ACTIVATION)
    y2, _ = functional(out, None, {}, [x, w], is_training=False, method="matmul")
    assert y2.abs().max() <= 0.5
