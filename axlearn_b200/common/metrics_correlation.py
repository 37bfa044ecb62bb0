"""Correlation metrics.

Parity targets in the reference (axlearn/common/metrics_correlation.py): ``matthews_corrcoef``
(:24), ``pearson_corrcoef`` (:71), ``spearman_corrcoef`` (:146, average ranks for ties).
"""

from __future__ import annotations

from typing import Optional

import torch

Tensor = torch.Tensor


def matthews_corrcoef(preds: Tensor, targets: Tensor, *, eps: float = 1e-8, mask: Optional[Tensor] = None) -> Tensor:
    """Binary Matthews correlation coefficient."""
    m = torch.ones_like(preds, dtype=torch.float32) if mask is None else mask.float()
    p, t = preds.float(), targets.float()
    tp = (m * p * t).sum()
    tn = (m * (1 - p) * (1 - t)).sum()
    fp = (m * p * (1 - t)).sum()
    fn = (m * (1 - p) * t).sum()
    den = torch.sqrt((tp + fp) * (tp + fn) * (tn + fp) * (tn + fn))
    return (tp * tn - fp * fn) / (den + eps)


def pearson_corrcoef(x: Tensor, y: Tensor, *, eps: float = 1e-8, mask: Optional[Tensor] = None) -> Tensor:
    m = torch.ones_like(x, dtype=torch.float32) if mask is None else mask.float()
    n = m.sum().clamp_min(1.0)
    x, y = x.float(), y.float()
    mx, my = (m * x).sum() / n, (m * y).sum() / n
    dx, dy = (x - mx) * m, (y - my) * m
    return (dx * dy).sum() / (torch.sqrt((dx * dx).sum() * (dy * dy).sum()) + eps)


def _rankdata(x: Tensor, mask: Tensor) -> Tensor:
    """1-based ranks among the unmasked entries, ties get the average rank."""
    big = torch.where(mask > 0, x.float(), torch.full_like(x.float(), float("inf")))
    less = (big[None, :] < big[:, None]).float() * mask[None, :]
    equal = (big[None, :] == big[:, None]).float() * mask[None, :]
    return less.sum(dim=1) + (equal.sum(dim=1) + 1) / 2


def spearman_corrcoef(x: Tensor, y: Tensor, *, eps: float = 1e-8, mask: Optional[Tensor] = None) -> Tensor:
    m = torch.ones_like(x, dtype=torch.float32) if mask is None else mask.float()
    return pearson_corrcoef(_rankdata(x, m), _rankdata(y, m), eps=eps, mask=m)
