"""LM head + softmax cross entropy evaluated chunk by chunk over tokens.

The ``[tokens, vocab]`` logits are the largest activation of a decoder-only LM (Fuji-7B:
16384 tokens x 32768 classes x 4 B = 2 GiB in fp32 per GPU).  This op never holds more than
one chunk of them: for each chunk it computes logits, the loss statistics and — in the same
pass — the gradient w.r.t. the logits, which is immediately folded into ``d_hidden`` and
``d_weight``.  Backward is then just a scale by the incoming scalar gradient.  The reference
gets the same memory behaviour from ``scan_chunk`` (axlearn/common/causal_lm.py:637-806) and,
on TPU, from its online-softmax kernel (axlearn/common/kernels/online_softmax_log_probs.py).

Loss definition (axlearn/common/loss.py:89-173, 298-321): per token ``ce = lse - logit[y]``,
``z = lse^2``; loss = sum(live * (ce + z_scale * z)) / denominator;
``dlogits = live/denominator * ((1 + 2*z_scale*lse) * softmax - onehot)``.
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.ops import dispatch


def _chunk_stats_and_grad(logits: torch.Tensor, targets: torch.Tensor, live: torch.Tensor,
                          z_loss_scale: float, inv_denom: torch.Tensor, need_grad: bool):
    """Returns (sum_ce, sum_z, sum_correct, dlogits or None). ``logits`` [n, V] may be
    overwritten."""
    if logits.is_cuda and not dispatch._flags.force_reference:  # pylint: disable=protected-access
        return dispatch._ops().ce_chunk(logits, targets, live, z_loss_scale, inv_denom, need_grad)
    lf = logits.float()
    v = lf.shape[-1]
    safe = targets.clamp(0, v - 1).long()
    lse = torch.logsumexp(lf, dim=-1)
    picked = torch.gather(lf, -1, safe[:, None]).squeeze(-1)
    livef = live.float()
    sum_ce = ((lse - picked) * livef).sum()
    sum_z = (lse * lse * livef).sum()
    sum_correct = ((lf.argmax(-1) == safe).float() * livef).sum()
    dlogits = None
    if need_grad:
        probs = torch.exp(lf - lse[:, None])
        dl = probs * (1.0 + 2.0 * z_loss_scale * lse)[:, None]
        dl.scatter_add_(1, safe[:, None], -torch.ones_like(lse)[:, None])
        dl = dl * (livef * inv_denom)[:, None]
        dlogits = dl.to(logits.dtype)
    return sum_ce, sum_z, sum_correct, dlogits


class _ChunkedLmHeadCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, live, z_loss_scale, denom, chunk_tokens, vocab_major):
        d = hidden.shape[-1]
        h2 = hidden.reshape(-1, d)
        t1 = targets.reshape(-1)
        l1 = live.reshape(-1)
        n = h2.shape[0]
        need_h = ctx.needs_input_grad[0]
        need_w = ctx.needs_input_grad[1]
        need_grad = need_h or need_w
        inv_denom = (1.0 / denom).to(torch.float32)
        w_vd = weight if vocab_major else weight.t()  # [V, D] view
        dh = torch.empty_like(h2) if need_h else None
        dw = torch.zeros(w_vd.shape, dtype=torch.float32, device=weight.device) if need_w else None
        sums = torch.zeros(3, dtype=torch.float32, device=hidden.device)
        for s in range(0, n, chunk_tokens):
            e = min(n, s + chunk_tokens)
            hc = h2[s:e]
            logits = dispatch.linear(hc, w_vd.t())
            ce, z, correct, dlogits = _chunk_stats_and_grad(
                logits, t1[s:e], l1[s:e], z_loss_scale, inv_denom, need_grad
            )
            sums += torch.stack([ce, z, correct])
            if need_h:
                dh[s:e] = dispatch.linear(dlogits, w_vd)
            if need_w:
                dw += dispatch.linear(dlogits.t(), hc).float()
        ce_mean = sums[0] * inv_denom
        z_mean = sums[1] * inv_denom
        acc = sums[2] * inv_denom
        loss = ce_mean + z_loss_scale * z_mean
        if need_grad:
            dw_out = None
            if need_w:
                dw_out = (dw if vocab_major else dw.t()).to(weight.dtype)
            ctx.save_for_backward(dh, dw_out)
            ctx.hidden_shape = hidden.shape
        ctx.mark_non_differentiable(ce_mean, z_mean, acc)
        return loss, ce_mean, z_mean, acc

    @staticmethod
    def backward(ctx, g_loss, *_):
        dh, dw = ctx.saved_tensors
        gh = None if dh is None else (dh * g_loss.to(dh.dtype)).reshape(ctx.hidden_shape)
        gw = None if dw is None else dw * g_loss.to(dw.dtype)
        return gh, gw, None, None, None, None, None, None


def chunked_lm_head_cross_entropy(
    hidden: torch.Tensor,
    weight: torch.Tensor,
    targets: torch.Tensor,
    *,
    live_targets: Optional[torch.Tensor] = None,
    z_loss_scale: float = 0.0,
    denominator: Optional[torch.Tensor] = None,
    chunk_tokens: int = 8192,
    weight_is_vocab_major: bool = True,
):
    vocab = weight.shape[0] if weight_is_vocab_major else weight.shape[1]
    if live_targets is None:
        live_targets = (targets >= 0) & (targets < vocab)
    num_live = live_targets.sum().to(torch.float32)
    denom = num_live.clamp_min(1.0) if denominator is None else denominator.to(torch.float32)
    loss, ce, z, acc = _ChunkedLmHeadCE.apply(
        hidden, weight, targets, live_targets, float(z_loss_scale), denom, int(chunk_tokens),
        bool(weight_is_vocab_major),
    )
    return loss, {"cross_entropy_loss": ce, "z_loss": z, "accuracy": acc, "num_live": num_live}
