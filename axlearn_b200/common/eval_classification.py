"""Precision / recall and ROC metrics of a classifier over a whole evaluation set.

Reference: axlearn/common/eval_classification.py:17-150 (``PrecisionRecallMetricCalculator``):
precision at fixed recall levels and recall at fixed precision levels, per label, from the scores
of all evaluation examples; here also the area under the ROC curve.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.evaler import GlobalMetricCalculator
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.metrics_classification import binary_classification_roc_auc_score, precision_recall_curve

Tensor = torch.Tensor


def precision_at_recall(y_true: Tensor, y_score: Tensor, recall_level: float, *, weight: Optional[Tensor] = None) -> Tensor:
    """The best precision among thresholds whose recall is at least ``recall_level``."""
    curve = precision_recall_curve(y_true, y_score, weight=weight)
    ok = curve["recalls"] >= recall_level
    return curve["precisions"][ok].max() if ok.any() else torch.tensor(0.0)


def recall_at_precision(y_true: Tensor, y_score: Tensor, precision_level: float, *, weight: Optional[Tensor] = None) -> Tensor:
    curve = precision_recall_curve(y_true, y_score, weight=weight)
    ok = curve["precisions"] >= precision_level
    return curve["recalls"][ok].max() if ok.any() else torch.tensor(0.0)


class PrecisionRecallMetricCalculator(GlobalMetricCalculator):
    """``model.predict`` must return ``{"logits": [B, labels]}``; ``input_batch["target_labels"]`` is
    ``[B, labels]`` multi-hot (entries < 0 are ignored)."""

    @config_class
    class Config(GlobalMetricCalculator.Config):
        label_names: Required[Sequence[str]] = REQUIRED
        precision_levels: Sequence[float] = ()
        recall_levels: Sequence[float] = ()
        metric_fn: Optional[object] = None

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        cfg = self._config
        scores = torch.cat([torch.sigmoid(o.predict_outputs["logits"].float()) for o in all_forward_outputs])
        labels = torch.cat([o.input_batch["target_labels"] for o in all_forward_outputs])
        out = {}
        for i, name in enumerate(cfg.label_names):
            live = labels[:, i] >= 0
            y, s, w = labels[live, i].clamp(0, 1), scores[live, i], None
            n = int(live.sum())
            for level in cfg.recall_levels:
                out[f"precision@recall{level}/{name}"] = WeightedSummary(precision_at_recall(y, s, level, weight=w), n)
            for level in cfg.precision_levels:
                out[f"recall@precision{level}/{name}"] = WeightedSummary(recall_at_precision(y, s, level, weight=w), n)
            if 0 < int(y.sum()) < n:
                out[f"roc_auc/{name}"] = WeightedSummary(binary_classification_roc_auc_score(y, s), n)
        return {self.formatted_metric_name(k): v for k, v in out.items()}
