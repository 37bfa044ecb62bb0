"""Image classification: backbone + linear head + softmax cross-entropy metrics.

Parity target in the reference: axlearn/vision/image_classification.py (``ImageClassificationModel``
:100 with ``ClassificationMetric`` :30: label smoothing, top-1 accuracy, optional top-5).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Linear
from axlearn_b200.common.metrics import WeightedSummary

Tensor = torch.Tensor


class ImageClassificationModel(BaseModel):
    """``input_batch = {"image": [B, H, W, C], "label": [B]}`` (labels < 0 are ignored)."""

    @config_class
    class Config(BaseModel.Config):
        backbone: Required[InstantiableConfig] = REQUIRED
        num_classes: Required[int] = REQUIRED
        classifier: InstantiableConfig = Linear.default_config().set(bias=True)
        label_smoothing: float = 0.0
        top_k: tuple = (1, 5)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("backbone", cfg.backbone)
        dim = self.backbone.endpoints_dims["embedding"]
        self._add_child("classifier", cfg.classifier.clone(input_dim=dim, output_dim=cfg.num_classes))

    def predict(self, input_batch: dict) -> dict:
        endpoints = self.backbone(input_batch["image"])
        return {"embedding": endpoints["embedding"], "logits": self.classifier(endpoints["embedding"])}

    def forward(self, input_batch: dict):
        cfg = self._config
        out = self.predict(input_batch)
        labels = input_batch["label"].long()
        live = labels >= 0
        n = live.sum().clamp_min(1)
        logits = out["logits"].float()
        per_example = F.cross_entropy(logits, labels.clamp_min(0), reduction="none", label_smoothing=cfg.label_smoothing)
        loss = (per_example * live).sum() / n
        self.add_summary("loss", WeightedSummary(loss.detach(), n))
        for k in cfg.top_k:
            if k <= cfg.num_classes:
                hit = (logits.topk(k, dim=-1).indices == labels[:, None]).any(dim=-1)
                self.add_summary(f"accuracy_top{k}" if k > 1 else "accuracy",
                                 WeightedSummary(((hit & live).sum() / n).detach(), n))
        return loss, out
