"""Plain PyTorch statements of every hot op.

These are the oracles: each CUDA kernel in ``axlearn_b200/csrc`` is tested against the
function of the same name here (evaluated in fp32), and they are the implementation that
runs on CPU.  Semantics follow the reference's layers:

* ``rms_norm``: axlearn/common/layers.py:374-417.
* ``rope`` (interleaved pairs, ``[sin | cos]`` tables): axlearn/common/attention.py:1063-1091,
  1301-1349.
* ``swiglu``: axlearn/common/attention.py:3354-3370 with activation ("nn.silu", "linear").
* ``attention`` (softmax(QKᵀ·scale + bias)V, fp32 softmax, GQA by head grouping):
  axlearn/common/flash_attention/common.py:487-535 and axlearn/common/attention.py:2107-2147.
* ``cross_entropy``: axlearn/common/loss.py:89-173, 234-327.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

NEG_INF = -0.7 * float(torch.finfo(torch.float32).max)


def rms_norm(x: torch.Tensor, scale: torch.Tensor, eps: float, *, upcast: bool = False) -> torch.Tensor:
    dt = x.dtype
    xf = x.float() if upcast else x
    moment2 = (xf * xf).mean(dim=-1, keepdim=True)
    y = xf * torch.rsqrt(moment2 + eps)
    return (y.to(dt) * scale.to(dt))


def layer_norm(x, scale, bias, eps: float) -> torch.Tensor:
    return F.layer_norm(x, x.shape[-1:], scale, bias, eps)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate) * up


def rope_tables(positions: torch.Tensor, dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """sin/cos of shape ``positions.shape + [dim/2]`` in fp32."""
    inv = theta ** (-torch.arange(0, dim, 2, device=positions.device, dtype=torch.float32) / dim)
    ang = positions.to(torch.float32).unsqueeze(-1) * inv
    return torch.sin(ang), torch.cos(ang)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float = 10000.0) -> torch.Tensor:
    """Rotary embedding over interleaved pairs ``(x[2i], x[2i+1])``.

    x: [B, T, N, H]; positions: [T] or [B, T].
    """
    h = x.shape[-1]
    sin, cos = rope_tables(positions, h, theta)  # [..., H/2]
    if sin.dim() == 2:
        sin, cos = sin[None], cos[None]
    sin = sin[:, :, None, :]
    cos = cos[:, :, None, :]
    xf = x.float()
    x0, x1 = xf[..., 0::2], xf[..., 1::2]
    y0 = x0 * cos - x1 * sin
    y1 = x1 * cos + x0 * sin
    return torch.stack([y0, y1], dim=-1).reshape(x.shape).to(x.dtype)


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    segment_ids: Optional[torch.Tensor] = None,
    kv_segment_ids: Optional[torch.Tensor] = None,
    sliding_window: Optional[int] = None,
    logit_cap: Optional[float] = None,
    q_offset: Optional[torch.Tensor] = None,
    dropout_mask: Optional[torch.Tensor] = None,
    return_probs: bool = False,
):
    """q: [B,T,N,H]; k,v: [B,S,Nkv,H]; bias broadcastable to [B,N,T,S] (additive).

    ``causal`` masks key position s > query position t (+ ``q_offset`` [B] when the queries
    are a suffix of the keys, as in decoding); ``sliding_window`` additionally masks
    s < t - window.
    """
    b, t, n, h = q.shape
    s, nkv = k.shape[1], k.shape[2]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(h)
    g = n // nkv
    qf = q.float().reshape(b, t, nkv, g, h)
    logits = torch.einsum("btkgh,bskh->bkgts", qf, k.float()) * softmax_scale
    logits = logits.reshape(b, n, t, s)
    if logit_cap:
        logits = logit_cap * torch.tanh(logits / logit_cap)
    if bias is not None:
        logits = logits + bias.float()
    mask = None
    if causal or sliding_window is not None:
        tpos = torch.arange(t, device=q.device)[None, :, None]
        if q_offset is not None:
            tpos = tpos + q_offset.reshape(-1, 1, 1)
        spos = torch.arange(s, device=q.device)[None, None, :]
        mask = torch.ones((1, t, s), dtype=torch.bool, device=q.device)
        if causal:
            mask = mask & (spos <= tpos)
        if sliding_window is not None:
            mask = mask & (spos >= tpos - sliding_window)
        mask = mask[:, None]
    if segment_ids is not None:
        kvseg = segment_ids if kv_segment_ids is None else kv_segment_ids
        seg = (segment_ids[:, :, None] == kvseg[:, None, :])[:, None]
        mask = seg if mask is None else (mask & seg)
    if mask is not None:
        logits = torch.where(mask, logits, torch.full_like(logits, NEG_INF))
    probs = torch.softmax(logits, dim=-1)
    if dropout_mask is not None:
        probs = probs * dropout_mask
    ctx = torch.einsum("bkgts,bskh->btkgh", probs.reshape(b, nkv, g, t, s), v.float())
    out = ctx.reshape(b, t, n, h).to(q.dtype)
    if return_probs:
        return out, probs
    return out


def cross_entropy(
    logits: torch.Tensor,
    targets: torch.Tensor,
    *,
    live_targets: Optional[torch.Tensor] = None,
    z_loss_scale: float = 0.0,
    denominator: Optional[torch.Tensor] = None,
):
    """Returns ``(loss, dict)`` where loss = mean over live targets of CE + z_scale·lse².

    ``denominator`` overrides the live-target count (used when the count is global across
    data-parallel ranks)."""
    lf = logits.float()
    num_classes = lf.shape[-1]
    if live_targets is None:
        live_targets = (targets >= 0) & (targets < num_classes)
    live = live_targets.to(torch.float32)
    safe = targets.clamp(0, num_classes - 1).long()
    lse = torch.logsumexp(lf, dim=-1)
    picked = torch.gather(lf, -1, safe.unsqueeze(-1)).squeeze(-1)
    per_token = lse - picked
    z = lse * lse
    denom = live.sum().clamp_min(1.0) if denominator is None else denominator
    ce = (per_token * live).sum() / denom
    zl = (z * live).sum() / denom
    loss = ce + z_loss_scale * zl
    correct = ((lf.argmax(-1) == safe).float() * live).sum() / denom
    return loss, {
        "cross_entropy_loss": ce,
        "z_loss": zl,
        "accuracy": correct,
        "per_token_loss": per_token * live,
        "num_live": live.sum(),
    }


def adamw_step(
    p: torch.Tensor,
    g: torch.Tensor,
    m: torch.Tensor,
    v: torch.Tensor,
    *,
    step: int,
    lr: float,
    b1: float,
    b2: float,
    eps: float,
    weight_decay: float,
    update_scale: float,
    grad_scale: float = 1.0,
) -> None:
    """In-place decoupled AdamW on fp32 tensors:
    ``p -= update_scale * (lr * m̂/(sqrt(v̂)+eps) + weight_decay * p)`` with the gradient
    pre-multiplied by ``grad_scale`` (global-norm clipping) and 1-based ``step``."""
    gf = g.float() * grad_scale
    m.mul_(b1).add_(gf, alpha=1 - b1)
    v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
    mhat = m / (1 - b1**step)
    vhat = v / (1 - b2**step)
    upd = lr * mhat / (vhat.sqrt() + eps) + weight_decay * p
    p.add_(upd, alpha=-update_scale)
