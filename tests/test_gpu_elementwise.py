"""Memory-bound kernels vs fp32 PyTorch references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"err {err} scale {scale}"


def _close_elementwise(out, ref, atol, rtol):
    diff = (out.float() - ref.float()).abs()
    bad = diff > atol + rtol * ref.float().abs()
    assert not bad.any(), f"{int(bad.sum())} elements off; worst {diff.max().item():.4g}"


@pytest.mark.parametrize("rows,d", [(333, 512), (100, 1024), (257, 2048), (1000, 4096), (9, 4096), (64, 768), (50, 8192)])
def test_fused_residual_rmsnorm_ops(rows, d):
    """``rms_norm_keep_input`` and ``add_rms_norm`` (warp-per-row kernels for the widths they take,
    the general kernel otherwise) against fp32 PyTorch, values and all gradients."""
    from axlearn_b200.ops import cuda_ops

    torch.manual_seed(4)
    eps = 1e-5

    def ref_norm(t, sc):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * sc

    x = torch.randn(rows, d, device="cuda").bfloat16().requires_grad_()
    r = torch.randn(rows, d, device="cuda").bfloat16().requires_grad_()
    scale = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16().requires_grad_()
    g_y, g_s = torch.randn(rows, d, device="cuda").bfloat16(), torch.randn(rows, d, device="cuda").bfloat16()

    # (x + r, norm(x + r)); loss takes both outputs.
    total, y = cuda_ops.add_rms_norm(x, r, scale, eps)
    (total.float() * g_s.float()).sum().backward(retain_graph=True)
    (y.float() * g_y.float()).sum().backward()
    xf, rf, sf = (t.detach().float().requires_grad_() for t in (x, r, scale))
    tf = (xf + rf).detach().bfloat16().float() + (xf + rf - (xf + rf).detach())   # value rounded to bf16, gradient of x + r
    yf = ref_norm(tf, sf)
    ((tf * g_s.float()).sum() + (yf * g_y.float()).sum()).backward()
    _close_elementwise(total, tf, 1e-6, 1e-6)
    _close_elementwise(y, yf, 0.03, 2e-2)
    _close_elementwise(x.grad, xf.grad, 0.06, 2e-2)
    assert torch.equal(x.grad, r.grad)
    _close(scale.grad, sf.grad, 2e-2)

    # (norm(x), x): the residual-branch gradient is added inside the backward kernel.
    x2 = x.detach().clone().requires_grad_()
    scale2 = scale.detach().clone().requires_grad_()
    y2, skip = cuda_ops.rms_norm_keep_input(x2, scale2, eps)
    ((y2.float() * g_y.float()).sum() + (skip.float() * g_s.float()).sum()).backward()
    x2f, s2f = x2.detach().float().requires_grad_(), scale2.detach().float().requires_grad_()
    ((ref_norm(x2f, s2f) * g_y.float()).sum() + (x2f * g_s.float()).sum()).backward()
    assert torch.equal(skip, x2)
    _close_elementwise(y2, ref_norm(x2f, s2f), 0.03, 2e-2)
    _close_elementwise(x2.grad, x2f.grad, 0.06, 2e-2)
    _close(scale2.grad, s2f.grad, 2e-2)
    torch.cuda.synchronize()
    cuda_ops.check_status()


@pytest.mark.parametrize("rows,d", [(64, 128), (1000, 4096), (37, 1024), (5000, 2048), (7, 512)])
def test_rmsnorm_fwd_bwd(rows, d):
    from axlearn_b200.ops import cuda_ops

    torch.manual_seed(0)
    x = torch.randn(rows, d, device="cuda").bfloat16().requires_grad_()
    scale = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16().requires_grad_()
    y = cuda_ops.rms_norm(x, scale, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xf, sf = x.detach().float().requires_grad_(), scale.detach().float().requires_grad_()
    yr = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-5) * sf
    yr.backward(g.float())
    _close(y, yr, 2e-2)
    _close(x.grad, xf.grad, 3e-2)
    _close(scale.grad, sf.grad, 3e-2)


def test_swiglu_fwd_bwd():
    from axlearn_b200.ops import cuda_ops

    torch.manual_seed(0)
    a = torch.randn(333, 1024, device="cuda").bfloat16().requires_grad_()
    b = torch.randn(333, 1024, device="cuda").bfloat16().requires_grad_()
    y = cuda_ops.swiglu(a, b)
    g = torch.randn_like(y)
    y.backward(g)
    af, bf = a.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    yr = torch.nn.functional.silu(af) * bf
    yr.backward(g.float())
    _close(y, yr, 2e-2)
    _close(a.grad, af.grad, 2e-2)
    _close(b.grad, bf.grad, 2e-2)


@pytest.mark.parametrize("b,t,n,h", [(2, 300, 4, 128), (3, 257, 32, 128), (1, 65, 5, 64), (2, 33, 3, 256), (1, 17, 2, 32),
                                     (1, 9, 1, 2048)])
def test_rope_fwd_bwd(b, t, n, h):
    from axlearn_b200.ops import cuda_ops, reference

    torch.manual_seed(0)
    x = torch.randn(b, t, n, h, device="cuda").bfloat16().requires_grad_()
    pos = torch.arange(t, device="cuda") + 3
    y = cuda_ops.rope(x, pos, 5e5)
    g = torch.randn_like(y)
    y.backward(g)
    xf = x.detach().float().requires_grad_()
    yr = reference.rope(xf, pos, 5e5)
    yr.backward(g.float())
    _close(y, yr, 2e-2)
    _close(x.grad, xf.grad, 2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy_fwd_bwd(dtype):
    from axlearn_b200.ops import cuda_ops, reference

    torch.manual_seed(0)
    n, v = 300, 32768
    logits = (3 * torch.randn(n, v, device="cuda")).to(dtype).requires_grad_()
    targets = torch.randint(0, v, (n,), device="cuda")
    targets[::7] = -1
    live = targets >= 0
    loss, aux = cuda_ops.cross_entropy(logits, targets, live_targets=live, z_loss_scale=1e-4)
    loss.backward()
    lf = logits.detach().float().requires_grad_()
    loss_r, aux_r = reference.cross_entropy(lf, targets, live_targets=live, z_loss_scale=1e-4)
    loss_r.backward()
    assert abs(loss.item() - loss_r.item()) < 2e-3 * abs(loss_r.item())
    assert abs(aux["accuracy"].item() - aux_r["accuracy"].item()) < 1e-6
    _close(logits.grad, lf.grad, 2e-2)


def test_chunked_lm_head_ce_matches_unfused():
    from axlearn_b200 import ops
    from axlearn_b200.ops import reference

    torch.manual_seed(0)
    n, d, v = 700, 256, 4096
    h = torch.randn(n, d, device="cuda").bfloat16().requires_grad_()
    w = (0.05 * torch.randn(v, d, device="cuda")).bfloat16().requires_grad_()
    t = torch.randint(0, v, (n,), device="cuda")
    loss, _ = ops.lm_head_cross_entropy(h, w, t, z_loss_scale=1e-4, chunk_tokens=256)
    loss.backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    loss_r, _ = reference.cross_entropy(hf @ wf.t(), t, z_loss_scale=1e-4)
    loss_r.backward()
    assert abs(loss.item() - loss_r.item()) < 5e-3 * abs(loss_r.item())
    _close(h.grad, hf.grad, 5e-2)
    _close(w.grad, wf.grad, 5e-2)


def test_adamw_and_sumsq():
    from axlearn_b200.ops import cuda_ops, reference

    torch.manual_seed(0)
    n = 1_000_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").bfloat16()
    m = torch.randn(n, device="cuda") * 0.1
    v = torch.rand(n, device="cuda") * 0.1
    shadow = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    scale = torch.tensor(0.5, device="cuda")
    cuda_ops.multi_tensor_adamw([p], [g], [m], [v], [shadow], [2.0], step=3, lr=1e-2, weight_decay=0.1,
                                b1=0.9, b2=0.95, eps=1e-8, grad_scale=scale)
    reference.adamw_step(pr, g, mr, vr, step=3, lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, weight_decay=0.2,
                         update_scale=1.0, grad_scale=0.5)
    _close(p, pr, 1e-5)
    _close(m, mr, 1e-5)
    _close(v, vr, 1e-5)
    assert torch.equal(shadow, p.bfloat16())
    ss = cuda_ops.sum_of_squares([g, p], [1.0, 0.5])
    ref = g.float().pow(2).sum() + 0.5 * p.pow(2).sum()
    assert abs(ss.item() - ref.item()) < 1e-4 * ref.item()
    assert ss.item() == cuda_ops.sum_of_squares([g, p], [1.0, 0.5]).item()
