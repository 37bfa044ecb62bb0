"""fp8 quantisers / block-scaled matmul emulation and the QuantizedDotGeneral layer (CPU)."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.common.quantized_dot_general.layers import DotGeneralQuantizationType, QuantizedDotGeneral
from axlearn_b200.ops import fp8_ops


def test_quantize_rows_roundtrip_error_is_fp8_sized():
    torch.manual_seed(0)
    x = (torch.randn(64, 256) * torch.logspace(-2, 2, 64)[:, None]).bfloat16()
    q, s = fp8_ops.quantize_rows(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (64, 2)
    back = fp8_ops.dequantize(q, s, row_gran=1)
    rel = (back - x.float()).abs() / x.float().abs().clamp_min(1e-6)
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 except near the block's underflow.
    big = x.float().abs() > 0.05 * x.float().abs().reshape(64, 2, 128).amax(-1).repeat_interleave(128, dim=1)
    assert rel[big].max() < 0.07
    # Each block uses the full range.
    assert torch.allclose(q.float().reshape(64, 2, 128).abs().amax(-1), torch.full((64, 2), 448.0))


def test_quantize_blocks_transpose_consistency():
    torch.manual_seed(1)
    x = torch.randn(200, 300).bfloat16()
    q, s = fp8_ops.quantize_blocks(x)
    qt, st = fp8_ops.quantize_blocks(x, transpose=True)
    assert q.shape == (200, 300) and s.shape == (2, 3) and qt.shape == (300, 200) and st.shape == (3, 2)
    assert torch.equal(qt.float(), q.float().t()) and torch.equal(st, s.t())
    q5, _ = fp8_ops.quantize_blocks(x, e5m2=True)
    assert q5.dtype == torch.float8_e5m2


def test_block_scaled_matmul_close_to_fp32():
    torch.manual_seed(2)
    x = torch.randn(256, 384).bfloat16()
    w = (torch.randn(384, 256) * 0.05).bfloat16()
    xq, sx = fp8_ops.quantize_rows(x)
    wq, sw = fp8_ops.quantize_blocks(w, transpose=True)
    y = fp8_ops.gemm_fp8(xq, wq, sx, sw, a_gran=1, out_dtype=torch.float32)
    ref = x.float() @ w.float()
    assert (y - ref).abs().max() < 0.06 * ref.abs().max()


def test_fp8_linear_gradients_track_bf16():
    torch.manual_seed(3)
    x = torch.randn(2, 128, 256).bfloat16().requires_grad_(True)
    w = (torch.randn(256, 384) * 0.05).bfloat16().requires_grad_(True)
    y = fp8_ops.fp8_linear(x, w)
    g = torch.randn_like(y)
    dx, dw = torch.autograd.grad(y, [x, w], g)
    yr = x.float() @ w.float()
    dxr, dwr = torch.autograd.grad(yr, [x, w], g.float())
    for a, b in ((y, yr), (dx, dxr), (dw, dwr)):
        assert (a.float() - b.float()).abs().max() < 0.08 * b.float().abs().max()


@pytest.mark.parametrize("scaling", ["block", "tensor"])
def test_quantized_dot_general_layer(scaling):
    cfg = QuantizedDotGeneral.default_config().set(name="q", scaling=scaling, fp8_amax_history_length=4)
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0))
    x = torch.randn(128, 256).bfloat16()
    w = (torch.randn(256, 128) * 0.1).bfloat16()
    y, oc = functional(layer, None, params, [x, w], is_training=True, method="matmul", drop_output_collections=())
    ref = x.float() @ w.float()
    assert (y.float() - ref).abs().max() < 0.1 * ref.abs().max()
    if scaling == "tensor":
        # Scales and amax histories are parameters; their new values come back as gradients
        # (tests/test_fp8_training.py covers the update through the learner).
        assert set(params) == {"input_scale", "kernel_scale", "output_grad_scale",
                               "input_amax_history", "kernel_amax_history", "output_grad_amax_history"}
        assert params["input_amax_history"].shape == (4,) and params["input_scale"].shape == ()
    else:
        assert params == {}


def test_int8_and_disabled():
    x = torch.randn(16, 32)
    w = torch.randn(32, 8)
    for qt in (DotGeneralQuantizationType.INT_8, None):
        layer = QuantizedDotGeneral.default_config().set(name="q", quantization_type=qt).instantiate(parent=None)
        y, _ = functional(layer, None, {}, [x, w], is_training=True, method="matmul")
        assert (y - x @ w).abs().max() < (0.2 if qt else 1e-5) * (x @ w).abs().max()
