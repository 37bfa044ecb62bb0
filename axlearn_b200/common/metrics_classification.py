"""Classification metrics on tensors.

Parity targets in the reference (axlearn/common/metrics_classification.py): ``confusion_matrix``
(:23), ``precision_recall_f_score`` (:56), ``f_score`` (:102), ``binary_clf_curve`` (:118),
``precision_recall_curve`` (:182), ``binary_classification_roc_auc_score`` (:234), ``roc_curve``
(:296), ``brier_score`` (:330).  All accept an optional ``weight`` (0 masks an example out).
"""

from __future__ import annotations

from typing import Optional

import torch

Tensor = torch.Tensor


def confusion_matrix(y_true: Tensor, y_pred: Tensor, *, num_classes: int, weight: Optional[Tensor] = None) -> Tensor:
    """``[num_classes, num_classes]``, rows = true class, columns = predicted class."""
    w = torch.ones_like(y_true, dtype=torch.float32) if weight is None else weight.float()
    flat = y_true.long() * num_classes + y_pred.long()
    return torch.zeros(num_classes * num_classes).index_add(0, flat.reshape(-1), w.reshape(-1)) \
        .reshape(num_classes, num_classes)


def precision_recall_f_score(y_true: Tensor, y_pred: Tensor, *, beta: float = 1.0, eps: float = 1e-8,
                             weight: Optional[Tensor] = None) -> dict:
    """Binary precision / recall / F-beta (labels and predictions in {0, 1})."""
    w = torch.ones_like(y_true, dtype=torch.float32) if weight is None else weight.float()
    t, p = y_true.float(), y_pred.float()
    tp = (w * t * p).sum()
    precision = tp / ((w * p).sum() + eps)
    recall = tp / ((w * t).sum() + eps)
    return dict(precision=precision, recall=recall, f_score=f_score(precision=precision, recall=recall, beta=beta, eps=eps))


def f_score(*, precision: Tensor, recall: Tensor, beta: float = 1.0, eps: float = 1e-8) -> Tensor:
    b2 = beta * beta
    return (1 + b2) * precision * recall / (b2 * precision + recall + eps)


def binary_clf_curve(y_true: Tensor, y_score: Tensor, *, weight: Optional[Tensor] = None):
    """Cumulative false / true positives at every distinct score threshold, scores descending.
    Returns ``(fps, tps, thresholds)``; masked examples count nothing."""
    w = torch.ones_like(y_score, dtype=torch.float32) if weight is None else weight.float()
    order = torch.argsort(y_score, descending=True, stable=True)
    s, t, w = y_score[order], y_true.float()[order], w[order]
    tps = torch.cumsum(t * w, 0)
    fps = torch.cumsum((1 - t) * w, 0)
    last_of_run = torch.ones_like(s, dtype=torch.bool)
    last_of_run[:-1] = s[1:] != s[:-1]
    return fps[last_of_run], tps[last_of_run], s[last_of_run]


def precision_recall_curve(y_true: Tensor, y_score: Tensor, *, weight: Optional[Tensor] = None) -> dict:
    fps, tps, thresholds = binary_clf_curve(y_true, y_score, weight=weight)
    precision = tps / (tps + fps).clamp_min(1e-12)
    recall = tps / tps[-1].clamp_min(1e-12)
    return dict(precisions=precision, recalls=recall, thresholds=thresholds)


def roc_curve(y_true: Tensor, y_score: Tensor, *, weight: Optional[Tensor] = None):
    """``(fpr, tpr, thresholds)`` starting at (0, 0)."""
    fps, tps, thresholds = binary_clf_curve(y_true, y_score, weight=weight)
    zero = fps.new_zeros(1)
    fps, tps = torch.cat([zero, fps]), torch.cat([zero, tps])
    thresholds = torch.cat([thresholds[:1] + 1, thresholds])
    return fps / fps[-1].clamp_min(1e-12), tps / tps[-1].clamp_min(1e-12), thresholds


def binary_classification_roc_auc_score(y_true: Tensor, y_score: Tensor, *, weight: Optional[Tensor] = None) -> Tensor:
    """Area under the ROC curve (trapezoids); 0 when only one class is present."""
    fpr, tpr, _ = roc_curve(y_true, y_score, weight=weight)
    w = torch.ones_like(y_score, dtype=torch.float32) if weight is None else weight.float()
    pos = (w * y_true.float()).sum()
    if pos == 0 or pos == w.sum():
        return fpr.new_zeros(())
    return torch.trapezoid(tpr, fpr)


def brier_score(labels: Tensor, logits: Tensor) -> Tensor:
    """Mean squared difference between sigmoid(logits) and binary labels."""
    return (torch.sigmoid(logits.float()) - labels.float()).square().mean()
