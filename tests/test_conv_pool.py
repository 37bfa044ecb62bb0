"""Convolution and pooling layers against torch.nn.functional / hand-written references."""

import pytest
import torch
import torch.nn.functional as F

from axlearn_b200.common import convolution, poolings, prng
from axlearn_b200.common.module import functional


def _run(cfg, *args, **kwargs):
    layer = cfg.set(name="l").instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0))
    out, _ = functional(layer, None, params, dict(zip(["x", "tokens"][:0], [])) or list(args), is_training=False) \
        if not kwargs else functional(layer, None, params, dict(kwargs), is_training=False)
    return layer, params, out


@pytest.mark.parametrize("padding,stride,dilation", [("SAME", 1, 1), ("VALID", 2, 1), ("CAUSAL", 1, 2), ("SAME", 2, 1)])
def test_conv1d(padding, stride, dilation):
    cfg = convolution.Conv1D.default_config().set(window=3, strides=stride, dilation=dilation, padding=padding,
                                                  input_dim=4, output_dim=6)
    x = torch.randn(2, 11, 4)
    layer, params, y = _run(cfg, x)
    assert list(y.shape) == layer.output_shape(input_shape=[2, 11, 4])
    (lo, hi), = layer._pad()  # pylint: disable=protected-access
    ref = F.conv1d(F.pad(x.transpose(1, 2), (lo, hi)), params["weight"].permute(2, 1, 0), params["bias"],
                   stride=stride, dilation=dilation).transpose(1, 2)
    assert torch.allclose(y, ref, atol=1e-5)
    if padding == "CAUSAL":
        x2 = x.clone()
        x2[:, 7:] += 1.0
        _, _, y2 = _run(cfg, x2)
        assert torch.allclose(y[:, :7], y2[:, :7], atol=1e-6)      # no look-ahead
    if padding == "SAME" and stride == 1:
        assert y.shape[1] == 11


def test_conv2d_depthwise_and_transpose_shapes():
    x = torch.randn(2, 8, 9, 4)
    cfg = convolution.Conv2D.default_config().set(window=(3, 3), strides=(2, 1), padding="SAME", input_dim=4,
                                                  output_dim=8, num_input_dim_groups=2)
    layer, params, y = _run(cfg, x)
    assert params["weight"].shape == (3, 3, 2, 8) and list(y.shape) == layer.output_shape(input_shape=[2, 8, 9, 4])
    dw = convolution.DepthwiseConv1D.default_config().set(window=5, padding="SAME", input_dim=4)
    _, p, y1 = _run(dw, torch.randn(2, 10, 4))
    assert p["weight"].shape == (5, 1, 4) and y1.shape == (2, 10, 4)
    tr = convolution.Conv2DTranspose.default_config().set(window=(3, 3), strides=(2, 2), input_dim=4, output_dim=5)
    _, _, yt = _run(tr, x)
    assert yt.shape == (2, 16, 18, 5)
    c3 = convolution.Conv3D.default_config().set(window=(2, 2, 2), input_dim=4, output_dim=3)
    _, _, y3 = _run(c3, torch.randn(1, 4, 5, 6, 4))
    assert y3.shape == (1, 3, 4, 5, 3)


def test_conv_with_paddings_and_stack_over_time():
    x = torch.randn(2, 10, 6, 3)
    paddings = torch.zeros(2, 10)
    paddings[1, 6:] = 1
    cfg = convolution.Conv2DWith1DPadding.default_config().set(window=(3, 3), strides=(2, 2), padding="SAME",
                                                               input_dim=3, output_dim=4)
    _, _, (y, p) = _run(cfg, x=x, paddings=paddings)
    assert y.shape[:2] == p.shape and p[0].sum() == 0 and p[1].sum() > 0
    assert (y[1][p[1] == 1] == 0).all()
    st = convolution.StackOverTime.default_config().set(stride=2)
    _, _, (ys, ps) = _run(st, x=torch.randn(2, 9, 5), paddings=torch.zeros(2, 9))
    assert ys.shape == (2, 4, 10) and ps.shape == (2, 4)


def test_poolings():
    tokens = torch.arange(2 * 5 * 3, dtype=torch.float32).reshape(2, 5, 3)
    paddings = torch.tensor([[0, 0, 0, 1, 1], [0, 0, 0, 0, 0]])
    mk = lambda klass, **kw: klass.default_config().set(input_dim=3, output_dim=3, **kw)
    _, _, avg = _run(mk(poolings.AveragePooling), tokens=tokens, paddings=paddings)
    assert torch.allclose(avg[0, 0], tokens[0, :3].mean(0)) and torch.allclose(avg[1, 0], tokens[1].mean(0))
    _, _, mx = _run(mk(poolings.MaxPooling), tokens=tokens, paddings=paddings)
    assert torch.equal(mx[0, 0], tokens[0, 2])
    _, _, first = _run(mk(poolings.FirstNTokenPooling, num_outputs=2), tokens=tokens, paddings=paddings)
    assert torch.equal(first, tokens[:, :2])
    _, _, last = _run(mk(poolings.LastNTokenPooling, num_outputs=2), tokens=tokens, paddings=paddings)
    assert torch.equal(last[0], tokens[0, 1:3]) and torch.equal(last[1], tokens[1, 3:5])
    _, _, att = _run(mk(poolings.AttentionPooling, num_outputs=2), tokens=tokens, paddings=paddings)
    assert att.shape == (2, 2, 3) and torch.isfinite(att).all()
