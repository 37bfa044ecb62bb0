"""Chunked ``extend_step`` of the causal convolutions reproduces the full-sequence ``forward``."""

import pytest
import torch

from axlearn_b200.audio.streaming.convolutions import (
    CausalConv1D,
    CausalConv1DTranspose,
    CausalConv1DWithPadding,
    CausalConv2DWith1DPadding,
    Conv1DTranspose,
)
from axlearn_b200.common import prng
from axlearn_b200.common.convolution import conv_explicit_padding
from axlearn_b200.common.module import functional


def _run(layer, params, method, *args, **kwargs):
    out, _ = functional(layer, None, params, kwargs if kwargs else list(args), is_training=False, method=method)
    return out


def test_explicit_padding_formulas():
    assert conv_explicit_padding("SAME", (5,), (2,), (1,)) == [(2, 2)]
    assert conv_explicit_padding("CAUSAL", (5,), (2,), (1,)) == [(3, 1)]
    assert conv_explicit_padding("CAUSAL", (5,), (2,), (2,)) == [(7, 1)]
    assert conv_explicit_padding("CAUSAL", (3, 3), (1, 2), (1, 1)) == [(2, 0), (1, 1)]
    assert conv_explicit_padding("VALID", (3, 3), (1, 1), (1, 1)) == [(0, 0), (0, 0)]


@pytest.mark.parametrize("window,stride,dilation,chunk", [(3, 1, 1, 1), (5, 2, 1, 4), (4, 2, 2, 2), (7, 3, 1, 6), (1, 1, 1, 3)])
def test_causal_conv1d_streams(window, stride, dilation, chunk):
    torch.manual_seed(0)
    cfg = CausalConv1D.default_config().set(name="c", window=window, strides=stride, dilation=dilation, input_dim=3, output_dim=5)
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0))
    t = 12 * stride
    x = torch.randn(2, t, 3)
    full = _run(layer, params, "forward", x)
    assert full.shape == (2, t // stride, 5)
    states = layer.init_states(batch_size=2)
    outs = []
    for start in range(0, t, chunk * stride if (chunk * stride) <= t else t):
        piece = x[:, start: start + chunk * stride]
        states, out = _run(layer, params, "extend_step", cached_states=states, input_data={"x": piece})
        outs.append(out["x"])
    assert torch.allclose(torch.cat(outs, dim=1), full, atol=1e-5)
    assert layer.cache_size() == (window - 1) * dilation + 1 - stride
    with pytest.raises(ValueError):
        if stride > 1:
            _run(layer, params, "extend_step", cached_states=states, input_data={"x": x[:, :1]})
        else:
            raise ValueError


def test_causal_conv1d_with_padding_streams():
    torch.manual_seed(1)
    cfg = CausalConv1DWithPadding.default_config().set(name="c", window=5, strides=2, input_dim=4, output_dim=4)
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(1))
    x = torch.randn(2, 16, 4)
    paddings = torch.zeros(2, 16)
    paddings[0, 11:] = 1
    paddings[1, 6:] = 1
    full, full_p = functional(layer, None, params, {"x": x, "paddings": paddings}, is_training=False)[0]
    assert full.shape == (2, 8, 4) and full_p.shape == (2, 8)
    assert full_p[0].tolist() == [0, 0, 0, 0, 0, 1, 1, 1] and (full[0, 5:] == 0).all()
    states = layer.init_states(batch_size=2)
    outs, ps = [], []
    for start in range(0, 16, 4):
        states, out = _run(layer, params, "extend_step", cached_states=states,
                           input_data={"x": x[:, start:start + 4], "paddings": paddings[:, start:start + 4]})
        outs.append(out["x"])
        ps.append(out["paddings"])
    assert torch.allclose(torch.cat(outs, dim=1), full, atol=1e-5)
    assert torch.equal(torch.cat(ps, dim=1).float(), full_p.float())


def test_causal_conv2d_streams():
    torch.manual_seed(2)
    cfg = CausalConv2DWith1DPadding.default_config().set(name="c", window=(3, 3), strides=(2, 2), input_dim=2, output_dim=3)
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(2))
    x = torch.randn(2, 12, 8, 2)
    paddings = torch.zeros(2, 12)
    paddings[1, 9:] = 1
    (full, full_p), _ = functional(layer, None, params, {"x": x, "paddings": paddings}, is_training=False)
    assert full.shape == (2, 6, 4, 3)
    states = layer.init_states(batch_size=2, feature_dim=8)
    outs, ps = [], []
    for start in range(0, 12, 4):
        states, out = _run(layer, params, "extend_step", cached_states=states,
                           input_data={"x": x[:, start:start + 4], "paddings": paddings[:, start:start + 4]})
        outs.append(out["x"])
        ps.append(out["paddings"])
    assert torch.allclose(torch.cat(outs, dim=1), full, atol=1e-5)
    assert torch.equal(torch.cat(ps, dim=1).float(), full_p.float())
    assert layer.cache_size() == 1 and layer.segment_pad() == 1 and layer.in_stride() == 2


@pytest.mark.parametrize("window,stride,chunk", [(4, 2, 2), (3, 1, 1), (5, 2, 3), (2, 2, 1), (6, 3, 2)])
def test_causal_conv1d_transpose_streams(window, stride, chunk):
    torch.manual_seed(3)
    cfg = CausalConv1DTranspose.default_config().set(name="c", window=window, strides=stride, input_dim=3, output_dim=2)
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(3))
    x = torch.randn(2, 6, 3)
    full = _run(layer, params, "forward", x)
    assert full.shape == (2, 6 * stride, 2)
    # Causality: output frames before t * stride do not depend on input t.
    x2 = x.clone()
    x2[:, 4:] += 1.0
    full2 = _run(layer, params, "forward", x2)
    assert torch.allclose(full[:, : 4 * stride], full2[:, : 4 * stride], atol=1e-6)
    states = layer.init_states(batch_size=2)
    outs = []
    for start in range(0, 6, chunk):
        states, out = _run(layer, params, "extend_step", cached_states=states, input_data={"x": x[:, start:start + chunk]})
        outs.append(out["x"])
    assert torch.allclose(torch.cat(outs, dim=1), full, atol=1e-5)


def test_conv1d_transpose_shapes():
    for padding, want in (("SAME", 12), ("VALID", 14), ("CAUSAL", 12)):
        cfg = Conv1DTranspose.default_config().set(name="t", window=4, strides=2, padding=padding, input_dim=3, output_dim=2)
        layer = cfg.instantiate(parent=None)
        params = layer.initialize_parameters_recursively(prng.PRNGKey(0))
        y = _run(layer, params, "forward", torch.randn(1, 6, 3))
        assert y.shape == (1, want, 2) and layer.output_shape(input_shape=[1, 6, 3]) == [1, want, 2]
