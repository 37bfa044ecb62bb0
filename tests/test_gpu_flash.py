"""tcgen05 flash attention forward/backward vs the fp32 reference attention."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"err {err} scale {scale}"


CASES = [
    # b, t, s, n, nkv, h, causal
    (1, 128, 128, 1, 1, 128, False),
    (2, 256, 256, 4, 4, 128, True),
    (1, 384, 384, 8, 2, 128, True),
    (2, 200, 200, 2, 1, 64, True),
    (1, 128, 320, 2, 2, 128, False),
    (1, 1024, 1024, 2, 2, 128, True),
    (1, 640, 640, 2, 1, 128, True),
    (2, 300, 300, 2, 2, 64, False),
]


@pytest.mark.parametrize("variant", ["v2", "v1"])
@pytest.mark.parametrize("b,t,s,n,nkv,h,causal", CASES)
def test_flash_fwd_bwd(b, t, s, n, nkv, h, causal, variant, monkeypatch):
    from axlearn_b200.ops import attention_ops, cuda_ops, flash_sm100, reference

    monkeypatch.setattr(flash_sm100, "FORWARD_VARIANT", variant)
    torch.manual_seed(0)
    q = torch.randn(b, t, n, h, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(b, s, nkv, h, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(b, s, nkv, h, device="cuda").bfloat16().requires_grad_()
    out = attention_ops.flash_attention(q, k, v, causal=causal, softmax_scale=None)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    cuda_ops.check_status()
    qf, kf, vf = (x.detach().float().requires_grad_() for x in (q, k, v))
    q_off = torch.full((b,), s - t, device="cuda") if s != t else None
    ref = reference.attention(qf, kf, vf, causal=causal, q_offset=q_off)
    ref.backward(g.float())
    _close(out, ref, 2e-2)
    _close(q.grad, qf.grad, 3e-2)
    _close(k.grad, kf.grad, 3e-2)
    _close(v.grad, vf.grad, 3e-2)


@pytest.mark.parametrize("variant", ["v2", "v1"])
def test_flash_large_scores_trigger_rescale(variant, monkeypatch):
    """Scores that grow along the key axis force the running-max rescale path."""
    from axlearn_b200.ops import attention_ops, flash_sm100, reference

    monkeypatch.setattr(flash_sm100, "FORWARD_VARIANT", variant)
    torch.manual_seed(0)
    b, t, n, h = 1, 512, 1, 128
    q = torch.randn(b, t, n, h, device="cuda").bfloat16()
    k = torch.randn(b, t, n, h, device="cuda")
    k = (k * torch.linspace(0.2, 4.0, t, device="cuda")[None, :, None, None]).bfloat16()
    v = torch.randn(b, t, n, h, device="cuda").bfloat16()
    out = attention_ops.flash_attention(q, k, v, causal=False, softmax_scale=None)
    ref = reference.attention(q.float(), k.float(), v.float(), causal=False)
    _close(out, ref, 2e-2)
