"""Loss functions.

Parity targets in the reference (axlearn/common/loss.py): ``cross_entropy`` (:89),
``binary_cross_entropy`` (:176), stable CE custom VJP (:234-327), ``mean_squared_error``
(:360), ``l1_loss`` (:419), contrastive losses (:442-720), ``focal_loss`` (:760),
``huber_loss`` (:810), ``flops_loss`` (:843), ``large_margin_cosine_loss`` (:887),
``giou_loss`` (:940), ``kl_divergence`` (:1052), ``koleo_loss`` (:1091),
``pairwise_loss``/``ranking_pairwise_loss`` (:1135, :1164).

The LM cross entropy runs through ``axlearn_b200.ops`` (fused softmax-CE kernels on GPU).
"""

from __future__ import annotations

import enum
from typing import Optional

import torch
import torch.nn.functional as F

from axlearn_b200 import ops

Tensor = torch.Tensor


class ReductionMethod(enum.Enum):
    NONE = None
    MEAN = "mean"
    SUM = "sum"


def _reduce(loss: Tensor, *, reduction: ReductionMethod, sample_weight: Optional[Tensor], eps: float = 0.0) -> Tensor:
    if reduction in (ReductionMethod.NONE, None):
        return loss
    if sample_weight is not None:
        w = sample_weight.to(loss.dtype)
        while w.dim() < loss.dim():
            w = w.unsqueeze(-1)
        loss = loss * w
        if reduction == ReductionMethod.MEAN:
            denom = w.expand_as(loss).sum()
            return loss.sum() / (denom + eps).clamp_min(eps or 1e-12)
    return loss.mean() if reduction == ReductionMethod.MEAN else loss.sum()


def cross_entropy(
    logits: Tensor,
    target_labels: Tensor,
    *,
    live_targets: Optional[Tensor] = None,
    z_loss_scale: float = 0.0,
    label_smoothing: float = 0.0,
    soft_target_labels: Optional[Tensor] = None,
    denominator: Optional[Tensor] = None,
) -> tuple[Tensor, dict]:
    """Softmax cross entropy + ``z_loss_scale * logsumexp^2``, averaged over live targets.

    Returns ``(loss, aux)`` with aux keys ``cross_entropy_loss``, ``z_loss``, ``accuracy``,
    ``num_live`` (and ``per_token_loss`` on the unfused path).
    """
    num_classes = logits.shape[-1]
    if live_targets is None:
        live_targets = (target_labels >= 0) & (target_labels < num_classes)
    if label_smoothing or soft_target_labels is not None:
        lf = logits.float()
        logp = torch.log_softmax(lf, dim=-1)
        if soft_target_labels is None:
            onehot = F.one_hot(target_labels.clamp(0, num_classes - 1).long(), num_classes).float()
            soft_target_labels = onehot * (1 - label_smoothing) + label_smoothing / num_classes
        live = live_targets.float()
        denom = live.sum().clamp_min(1.0) if denominator is None else denominator
        per = -(soft_target_labels * logp).sum(-1)
        lse = torch.logsumexp(lf, dim=-1)
        ce = (per * live).sum() / denom
        z = (lse * lse * live).sum() / denom
        acc = ((lf.argmax(-1) == target_labels).float() * live).sum() / denom
        return ce + z_loss_scale * z, {
            "cross_entropy_loss": ce, "z_loss": z, "accuracy": acc,
            "per_token_loss": per * live, "num_live": live.sum(),
        }
    return ops.cross_entropy(
        logits, target_labels, live_targets=live_targets, z_loss_scale=z_loss_scale, denominator=denominator
    )


def binary_cross_entropy(
    logits: Tensor, *, target_labels: Tensor, live_targets: Optional[Tensor] = None
) -> tuple[Tensor, dict]:
    if live_targets is None:
        live_targets = (target_labels == 0) | (target_labels == 1)
    live = live_targets.float()
    per = F.binary_cross_entropy_with_logits(logits.float(), target_labels.clamp(0, 1).float(), reduction="none")
    denom = live.sum().clamp_min(1.0)
    loss = (per * live).sum() / denom
    return loss, {"binary_cross_entropy_loss": loss, "per_target_loss": per * live}


def mean_squared_error(preds: Tensor, targets: Tensor, sample_weight: Optional[Tensor] = None,
                       reduction: ReductionMethod = ReductionMethod.MEAN, eps: float = 0.0) -> Tensor:
    return _reduce((preds.float() - targets.float()) ** 2, reduction=reduction, sample_weight=sample_weight, eps=eps)


def l1_loss(preds: Tensor, targets: Tensor, sample_weight: Optional[Tensor] = None,
            reduction: ReductionMethod = ReductionMethod.MEAN, eps: float = 0.0) -> Tensor:
    return _reduce((preds.float() - targets.float()).abs(), reduction=reduction, sample_weight=sample_weight, eps=eps)


def huber_loss(*, predictions: Tensor, targets: Tensor, delta: float = 1.0,
               reduce_axis: Optional[int] = None, sample_weight: Optional[Tensor] = None,
               reduction: ReductionMethod = ReductionMethod.MEAN) -> Tensor:
    err = (predictions.float() - targets.float()).abs()
    quad = torch.clamp(err, max=delta)
    loss = 0.5 * quad**2 + delta * (err - quad)
    if reduce_axis is not None:
        loss = loss.mean(dim=reduce_axis)
    return _reduce(loss, reduction=reduction, sample_weight=sample_weight)


def focal_loss(logits: Tensor, *, targets: Tensor, alpha: float = 0.25, gamma: float = 2.0,
               sample_weight: Optional[Tensor] = None, reduction: ReductionMethod = ReductionMethod.MEAN) -> Tensor:
    lf = logits.float()
    t = targets.float()
    bce = F.binary_cross_entropy_with_logits(lf, t, reduction="none")
    p = torch.sigmoid(lf)
    pt = p * t + (1 - p) * (1 - t)
    w = (1 - pt) ** gamma
    if alpha >= 0:
        w = w * (alpha * t + (1 - alpha) * (1 - t))
    return _reduce(w * bce, reduction=reduction, sample_weight=sample_weight)


def kl_divergence(log_predictions: Tensor, targets: Tensor, is_log_targets: bool = False) -> tuple[Tensor, dict]:
    lp = log_predictions.float()
    if is_log_targets:
        per = (targets.float().exp() * (targets.float() - lp)).sum(-1)
    else:
        t = targets.float()
        per = torch.where(t > 0, t * (t.clamp_min(1e-30).log() - lp), torch.zeros_like(t)).sum(-1)
    loss = per.mean()
    return loss, {"per_example_loss": per}


def contrastive_logits(x: Tensor, y: Tensor) -> Tensor:
    """Pairwise similarities ``x @ y^T`` of L2-normalised embeddings."""
    return x @ y.t()


def symmetric_contrastive_loss_from_logits(
    x_y_logits: Tensor, y_x_logits: Tensor, *, temperature: float = 1.0,
    y_as_key_weight: float = 0.5,
) -> Tensor:
    n = x_y_logits.shape[0]
    labels = torch.arange(n, device=x_y_logits.device)
    l_xy = F.cross_entropy(x_y_logits.float() / temperature, labels)
    l_yx = F.cross_entropy(y_x_logits.float() / temperature, labels)
    return y_as_key_weight * l_xy + (1 - y_as_key_weight) * l_yx


def asymmetric_contrastive_loss_from_logits(logits: Tensor, *, key_paddings: Optional[Tensor] = None,
                                            temperature: float = 1.0, soft_labels: Optional[Tensor] = None) -> Tensor:
    lf = logits.float() / temperature
    if key_paddings is not None:
        lf = lf + key_paddings.float()[None, :] * (-1e9)
    n = lf.shape[0]
    if soft_labels is None:
        return F.cross_entropy(lf, torch.arange(n, device=lf.device))
    return -(soft_labels * torch.log_softmax(lf, -1)).sum(-1).mean()


def flops_loss(*, embeddings: Tensor, paddings: Optional[Tensor] = None, sparsity_threshold: float = 0.0):
    """FLOPs regulariser of sparse embeddings ``sum_j (mean_i |e_ij|)^2`` over the live rows
    (reference: axlearn/common/loss.py:843).  Returns ``(loss, average_sparsity_count)``: the
    second is the mean number of entries per live row with ``|e| <= sparsity_threshold``."""
    if embeddings.dim() == 3:
        if embeddings.shape[1] != 1:
            raise ValueError("expected [batch, 1, dim] or [batch, dim]")
        embeddings = embeddings.squeeze(1)
    e = embeddings.float().abs()
    live = torch.ones(e.shape[0], device=e.device) if paddings is None else 1 - paddings.float().reshape(-1)
    n = live.sum()
    sparsity = ((e <= sparsity_threshold).float().sum(-1) * live).sum() / n
    mean = (e * live[:, None]).sum(0) / n
    return (mean ** 2).sum(), sparsity


def large_margin_cosine_loss(logits: Tensor, *, labels: Tensor, alpha: float = 1.0, margin: float = 0.0):
    num_classes = logits.shape[-1]
    onehot = F.one_hot(labels.long(), num_classes).float()
    adj = alpha * (logits.float() - margin * onehot)
    return cross_entropy(adj, labels)


def giou_loss(*, predictions: Tensor, targets: Tensor, eps: float = 1e-7,
              reduction: ReductionMethod = ReductionMethod.MEAN, sample_weight=None) -> Tensor:
    """Generalised IoU loss on boxes ``[..., (y1, x1, y2, x2)]``."""
    p, t = predictions.float(), targets.float()
    area = lambda b: (b[..., 2] - b[..., 0]).clamp_min(0) * (b[..., 3] - b[..., 1]).clamp_min(0)
    iy1, ix1 = torch.max(p[..., 0], t[..., 0]), torch.max(p[..., 1], t[..., 1])
    iy2, ix2 = torch.min(p[..., 2], t[..., 2]), torch.min(p[..., 3], t[..., 3])
    inter = (iy2 - iy1).clamp_min(0) * (ix2 - ix1).clamp_min(0)
    union = area(p) + area(t) - inter
    iou = inter / (union + eps)
    ey1, ex1 = torch.min(p[..., 0], t[..., 0]), torch.min(p[..., 1], t[..., 1])
    ey2, ex2 = torch.max(p[..., 2], t[..., 2]), torch.max(p[..., 3], t[..., 3])
    enclose = (ey2 - ey1).clamp_min(0) * (ex2 - ex1).clamp_min(0)
    giou = iou - (enclose - union) / (enclose + eps)
    return _reduce(1 - giou, reduction=reduction, sample_weight=sample_weight)


def koleo_loss(embeddings: Tensor, *, eps: float = 1e-8, normalize_embedding: bool = True) -> Tensor:
    """Kozachenko-Leonenko differential-entropy regulariser (spreads embeddings; reference:
    axlearn/common/loss.py:1091-1132): ``-mean(log(distance to the nearest other embedding))``, the
    neighbour being picked by largest dot product."""
    e = embeddings.float()
    if normalize_embedding:
        e = l2_normalize(e, eps=eps)
    dots = e @ e.t()
    dots.fill_diagonal_(-1)
    nearest = dots.argmax(dim=-1)
    distances = torch.sqrt(((e[nearest] - e + eps) ** 2).sum(dim=-1))
    return -torch.log(distances + eps).mean()


def pairwise_loss(*, logits: Tensor, pair_weights: Tensor, loss_scale: Optional[Tensor] = None):
    """Weighted mean over pairs ``(i, j)`` of ``softplus(-(logit_i - logit_j))`` (reference:
    axlearn/common/loss.py:1135).  ``pair_weights [batch, docs, docs]``; ``loss_scale [batch]``.
    Returns ``(mean_loss, total_weight)``."""
    lf = logits.float()
    diff = lf[..., :, None] - lf[..., None, :]
    w = pair_weights.float()
    labels = (w > 0).float()
    per = F.binary_cross_entropy_with_logits(diff, labels, reduction="none") * w
    if loss_scale is not None:
        per = per * torch.as_tensor(loss_scale, dtype=per.dtype, device=per.device).reshape(-1, 1, 1)
    total = w.sum()
    return per.sum() / (1e-8 + total), total


def ranking_pairwise_loss(*, logits: Tensor, ranks: Tensor, loss_scale: Optional[Tensor] = None):
    """Pairs (i, j) with ``0 < rank_i < rank_j`` should have ``logit_i > logit_j`` (reference:
    axlearn/common/loss.py:1164).  Returns ``(mean_loss, number of pairs)``."""
    ranked = ranks > 0
    w = (ranked[..., :, None] & (ranks[..., :, None] < ranks[..., None, :])).float()
    return pairwise_loss(logits=logits, pair_weights=w, loss_scale=loss_scale)


def l2_normalize(x: Tensor, eps: float = 1e-8, dim: int = -1) -> Tensor:
    """``x / max(||x||, eps)`` (reference: axlearn/common/normalize.py ``l2_normalize``: the sum of
    squares is floored at ``eps^2`` before the square root)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().sum(dim=dim, keepdim=True).clamp_min(eps * eps))).to(x.dtype)


def negative_cosine_similarity_loss(predictions: Tensor, targets: Tensor, *, normalize_embedding: bool = True,
                                    eps: float = 1e-8, live_targets: Optional[Tensor] = None,
                                    reduction: ReductionMethod = ReductionMethod.MEAN) -> tuple[Tensor, dict]:
    """``-mean(cos(predictions, targets))`` over live positions (reference:
    axlearn/common/loss.py:1007-1050); aux holds the per-position and per-element similarities."""
    if normalize_embedding:
        targets = l2_normalize(targets, eps=eps)
        predictions = l2_normalize(predictions, eps=eps)
    elementwise = targets * predictions
    cosine = elementwise.sum(dim=-1)
    loss = -_reduce(cosine, reduction=reduction, sample_weight=live_targets)
    return loss, {"cosine_similarity": cosine, "elementwise_similarity": elementwise}


def sigmoid_cross_entropy_with_logits(logits: Tensor, targets: Tensor) -> Tensor:
    """Element-wise ``max(x, 0) - x z + log(1 + exp(-|x|))``."""
    return F.binary_cross_entropy_with_logits(logits.float(), targets.float(), reduction="none")


def categorical_hinge_loss(logits: Tensor, targets: Tensor) -> Tensor:
    """``max(0, max((1 - targets) * logits) - sum(targets * logits) + 1)`` per example."""
    pos = (targets * logits).sum(dim=-1)
    neg = ((1.0 - targets) * logits).amax(dim=-1)
    return torch.clamp(neg - pos + 1.0, min=0.0)


def bilinear_mean_squared_error(preds: Tensor, targets: Tensor, *, shape: tuple, sample_weight: Optional[Tensor] = None,
                                eps: float = 1e-7) -> Tensor:
    """Mean squared error after bilinearly resizing ``preds - targets`` (``[B, H, W, C]``) to
    ``shape`` (reference: :383-417)."""
    diff = (preds - targets).float()
    src = diff.shape
    for d, n in zip(src, shape):
        if not (d % n == 0 or n % d == 0):
            raise NotImplementedError(f"dims of shape and (preds - targets).shape must divide one another: {tuple(src)} vs {shape}")
    diff = F.interpolate(diff.permute(0, 3, 1, 2), size=tuple(shape[1:3]), mode="bilinear", align_corners=False,
                         antialias=False).permute(0, 2, 3, 1)
    return _reduce(diff.square(), reduction=ReductionMethod.MEAN, sample_weight=sample_weight, eps=eps)


def asymmetric_contrastive_loss_from_features(queries: Tensor, positive_keys: Tensor, *, negative_keys: Optional[Tensor] = None,
                                              temperature: float = 1.0, **kwargs) -> Tensor:
    """Contrastive loss of each query against its positive key and all other (+ extra negative)
    keys; features are expected to be normalised by the caller."""
    keys = positive_keys if negative_keys is None else torch.cat([positive_keys, negative_keys], dim=0)
    return asymmetric_contrastive_loss_from_logits(contrastive_logits(queries, keys) / temperature, **kwargs)


def symmetric_contrastive_loss_from_features(x: Tensor, y: Tensor, *, temperature: float = 1.0, **kwargs) -> Tensor:
    return symmetric_contrastive_loss_from_logits(contrastive_logits(x, y) / temperature, **kwargs)
