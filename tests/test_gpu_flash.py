"""tcgen05 flash attention forward / backward vs the fp32 reference attention."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol, what=""):
    """Max-norm check plus a per-element ``atol + rtol * |ref|`` check (an error confined to
    small-magnitude outputs or to one tile edge passes the first but not the second)."""
    a, b = a.float(), b.float()
    err = (a - b).abs()
    scale = b.abs().max().item() + 1e-6
    assert err.max().item() / scale < tol, f"{what}: err {err.max().item()} scale {scale}"
    bound = 0.75 * tol * scale + 4 * tol * b.abs()
    bad = (err > bound).sum().item()
    assert bad == 0, f"{what}: {bad} elements outside atol + rtol * |ref|"


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
    (1, 4096, 4096, 2, 2, 128, True),
    (1, 8192, 8192, 1, 1, 128, True),
]

# (forward variant, backward variant): the defaults, and the older kernels kept as cross-checks.
VARIANTS = [("v3", "fused"), ("v2", "split"), ("v1", "split")]


def _run(q, k, v, causal, **masks):
    from axlearn_b200.ops import attention_ops, cuda_ops, reference

    out = attention_ops.flash_attention(q, k, v, causal=causal, softmax_scale=None, **masks)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    cuda_ops.check_status()
    qf, kf, vf = (x.detach().float().requires_grad_() for x in (q, k, v))
    t, s = q.shape[1], k.shape[1]
    q_off = torch.full((q.shape[0],), s - t, device="cuda") if s != t else None
    ref = reference.attention(qf, kf, vf, causal=causal, q_offset=q_off, **masks)
    ref.backward(g.float())
    _close(out, ref, 2e-2, "out")
    _close(q.grad, qf.grad, 3e-2, "dq")
    _close(k.grad, kf.grad, 3e-2, "dk")
    _close(v.grad, vf.grad, 3e-2, "dv")


def _qkv(b, t, s, n, nkv, h):
    q = torch.randn(b, t, n, h, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(b, s, nkv, h, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(b, s, nkv, h, device="cuda").bfloat16().requires_grad_()
    return q, k, v


@pytest.mark.parametrize("fwd,bwd", VARIANTS)
@pytest.mark.parametrize("b,t,s,n,nkv,h,causal", CASES)
def test_flash_fwd_bwd(b, t, s, n, nkv, h, causal, fwd, bwd, monkeypatch):
    from axlearn_b200.ops import flash_sm100

    if t > 2048 and fwd != "v3":
        pytest.skip("long sequences are checked on the default kernels only")
    monkeypatch.setattr(flash_sm100, "FORWARD_VARIANT", fwd)
    monkeypatch.setattr(flash_sm100, "BACKWARD_VARIANT", bwd)
    torch.manual_seed(0)
    _run(*_qkv(b, t, s, n, nkv, h), causal)


def _packed_segments(b, t, pieces):
    cuts = torch.sort(torch.randint(1, t, (b, pieces - 1), device="cuda"), dim=1).values
    return (torch.arange(t, device="cuda")[None, :, None] >= cuts[:, None, :]).sum(-1).to(torch.int32)


MASK_CASES = [
    # b, t, n, nkv, h, causal, window, cap, segments
    (2, 512, 2, 2, 128, True, None, None, 4),
    (1, 1024, 2, 1, 128, True, 200, None, 0),
    (1, 768, 2, 2, 128, True, None, 30.0, 0),
    (2, 640, 4, 2, 64, True, 100, 20.0, 3),
    (1, 512, 2, 2, 128, False, None, None, 5),
    (1, 2048, 2, 2, 128, True, 300, None, 6),
    (1, 333, 2, 2, 128, True, 50, None, 2),
    (1, 8192, 1, 1, 128, True, 1024, None, 9),
]


@pytest.mark.parametrize("b,t,n,nkv,h,causal,window,cap,pieces", MASK_CASES)
def test_flash_segment_ids_window_and_logit_cap(b, t, n, nkv, h, causal, window, cap, pieces):
    """Packed sequences (segment ids), sliding windows and the tanh logit cap run inside the
    kernels, forward and backward."""
    torch.manual_seed(1)
    segs = _packed_segments(b, t, pieces) if pieces else None
    _run(*_qkv(b, t, t, n, nkv, h), causal, segment_ids=segs, sliding_window=window, logit_cap=cap)


def test_unsorted_segment_ids():
    """Ids need not be sorted: tile skipping only uses per-tile [min, max] ranges."""
    torch.manual_seed(2)
    b, t = 2, 640
    segs = torch.randint(0, 3, (b, t), device="cuda", dtype=torch.int32)
    _run(*_qkv(b, t, t, 2, 2, 128), True, segment_ids=segs)


def test_shape_fuzz():
    """Seeded random shapes, including lengths that are not multiples of the 128-row tiles."""
    import random

    rng = random.Random(0)
    for _ in range(8):
        h = rng.choice([64, 128])
        nkv = rng.choice([1, 2])
        n = nkv * rng.choice([1, 2, 4])
        t = rng.randint(1, 900)
        causal = rng.random() < 0.7
        s = t if causal or rng.random() < 0.5 else rng.randint(1, 900)
        torch.manual_seed(t)
        _run(*_qkv(rng.choice([1, 2]), t, s, n, nkv, h), causal)


def test_dispatch_routes_masks_to_the_kernel(monkeypatch):
    """``ops.attention`` with segment ids / window / cap must not fall back to the [T, S] path."""
    from axlearn_b200 import ops
    from axlearn_b200.ops import reference

    def boom(*a, **k):
        raise AssertionError("materialised attention path used")

    monkeypatch.setattr(reference, "attention", boom)
    q, k, v = _qkv(1, 256, 256, 2, 2, 128)
    segs = _packed_segments(1, 256, 2)
    out = ops.attention(q, k, v, causal=True, segment_ids=segs, sliding_window=64, logit_cap=50.0)
    assert out.shape == q.shape


@pytest.mark.parametrize("variant", ["v3", "v2", "v1"])
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


def test_remat_policy_skips_attention_forward_in_replay():
    """With the default save policy the replay reuses the kept context / log-sum-exp: the forward
    kernel runs once per layer and step, and gradients equal those of full rematerialisation."""
    from axlearn_b200.common import prng, remat
    from axlearn_b200.common.attention import RematRegexSavePatterns
    from axlearn_b200.common.base_layer import RematSpec, nothing_saveable
    from axlearn_b200.common.module import functional
    from axlearn_b200.common.utils import flatten_items, tree_map
    from axlearn_b200.experiments.text.gpt import fuji
    from axlearn_b200.ops import flash_sm100

    def grads(spec):
        cfg = fuji.model_config(num_layers=2, hidden_dim=256, num_heads=2, num_kv_heads=None, vocab_size=512,
                                rope_theta=1e4, shared_lm_head=True, ffn_dim=512)
        cfg.decoder.transformer.layer.remat_spec = spec
        cfg.name = "model"
        model = cfg.instantiate(parent=None)
        params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cuda")
        params = tree_map(lambda t: t.bfloat16().requires_grad_(), params)
        torch.manual_seed(0)
        ids = torch.randint(0, 512, (2, 257), device="cuda")
        batch = {"input_ids": ids[:, :-1], "target_labels": ids[:, 1:]}
        calls = {"n": 0}
        real = flash_sm100.forward

        def counting(*a, **k):
            calls["n"] += 1
            return real(*a, **k)

        flash_sm100.forward = counting
        try:
            (loss, _), _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=True, method="forward")
            loss.backward()
        finally:
            flash_sm100.forward = real
        torch.cuda.synchronize()
        return calls["n"], loss.detach(), [t.grad.float() for _, t in flatten_items(params)]

    n_full, loss_full, g_full = grads(RematSpec(policy=nothing_saveable))
    n_sel, loss_sel, g_sel = grads(RematSpec(policy=remat.save_only_these_names_regex(
        RematRegexSavePatterns.NATIVE_ATTENTION.value)))
    assert n_full == 4 and n_sel == 2
    assert torch.equal(loss_full, loss_sel)
    for a, b in zip(g_full, g_sel):
        _close(a, b, 2e-2, "grad")
