"""GLUE / SuperGLUE task metrics over a whole evaluation set.

Reference: axlearn/common/metrics_glue.py (``GLUEMetricAccumulator`` :17, ``GLUEMetricCalculator``
:62, ``glue_metrics`` :124-181).  Correlation metrics (STS-B) cannot be averaged over batches, so
predictions and labels of every batch are kept and the metrics are computed once at the end:
accuracy for every classification task, plus Matthews correlation for CoLA, F1 for MRPC / QQP /
ReCoRD, and Pearson / Spearman correlation for STS-B.
"""

from __future__ import annotations

from typing import Optional, Union

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.evaler import BaseMetricCalculator
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.metrics_classification import precision_recall_f_score
from axlearn_b200.common.metrics_correlation import matthews_corrcoef, pearson_corrcoef, spearman_corrcoef

Tensor = torch.Tensor


def glue_metrics(*, task: str, target_labels: Tensor, preds: Tensor, mask: Tensor) -> dict:
    out = {}
    live = mask.bool()
    n = live.sum()
    if task == "stsb":
        out["pearson_corr"] = WeightedSummary(pearson_corrcoef(preds.float(), target_labels.float(), mask=live), n)
        out["spearman_corr"] = WeightedSummary(spearman_corrcoef(preds.float(), target_labels.float(), mask=live), n)
    else:
        out["accuracy"] = WeightedSummary(((preds == target_labels) & live).sum() / n.clamp_min(1), n)
    if task == "cola":
        out["matthews_corr"] = WeightedSummary(matthews_corrcoef(preds, target_labels, mask=live), n)
    elif task in ("mrpc", "qqp", "record"):
        # A prediction outside {0, 1} counts as the wrong class.
        invalid = (preds != 0) & (preds != 1)
        fixed = torch.where(invalid, 1 - target_labels, preds)
        out["f1"] = WeightedSummary(
            precision_recall_f_score(target_labels, fixed, beta=1.0, weight=live.float())["f_score"], n)
    return out


class GLUEMetricCalculator(BaseMetricCalculator):
    """Runs ``model.forward`` per batch (its aux outputs must hold ``logits``) and computes the
    task's metrics over all batches."""

    @config_class
    class Config(BaseMetricCalculator.Config):
        task: Required[str] = REQUIRED
        ignore_target_label: Required[Union[int, float]] = REQUIRED
        model_method: str = "forward"
        model_method_kwargs: dict = {}

    def init_state(self, *, prng_key, model_params):
        return {"prng_key": prng_key}

    def forward(self, input_batch, *, model_params, state):
        cfg = self._config
        key, next_key = prng.split(state["prng_key"], 2)
        (loss, aux), _ = self._call_model(method=cfg.model_method, prng_key=key, model_params=model_params,
                                          input_batch=input_batch, **cfg.model_method_kwargs)
        logits = aux["logits"]
        labels = input_batch["target_labels"]
        preds = logits.squeeze(-1) if cfg.task == "stsb" else logits.argmax(dim=-1)
        live = labels != cfg.ignore_target_label
        return {"state": {"prng_key": next_key},
                "output": dict(preds=preds.cpu(), target_labels=labels.cpu(), mask=live.cpu(),
                               loss=float(loss) * int(live.sum()))}

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        cat = lambda k: torch.cat([o[k].reshape(-1) for o in all_forward_outputs])
        mask = cat("mask")
        out = glue_metrics(task=self._config.task, target_labels=cat("target_labels"), preds=cat("preds"), mask=mask)
        n = mask.sum()
        out["loss"] = WeightedSummary(torch.tensor(sum(o["loss"] for o in all_forward_outputs)) / n.clamp_min(1), n)
        return {self.formatted_metric_name(k): v for k, v in out.items()}
