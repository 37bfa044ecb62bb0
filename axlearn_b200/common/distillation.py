"""Knowledge distillation.

Parity target in the reference: axlearn/common/distillation.py (``DistillationModel`` :30: a
frozen ``teacher`` and a ``student`` see the same batch; the loss combines the student's own loss
with a soft-target term between the two logit distributions).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class

Tensor = torch.Tensor


def soft_target_kl(*, student_logits: Tensor, teacher_logits: Tensor, temperature: float = 1.0,
                   live: Tensor = None) -> Tensor:
    """``T^2 * KL(softmax(teacher / T) || softmax(student / T))`` averaged over live positions."""
    t = temperature
    log_p_s = F.log_softmax(student_logits.float() / t, dim=-1)
    p_t = F.softmax(teacher_logits.float() / t, dim=-1)
    kl = (p_t * (torch.log(p_t.clamp_min(1e-30)) - log_p_s)).sum(dim=-1)
    if live is None:
        return kl.mean() * t * t
    live = live.float()
    return (kl * live).sum() / live.sum().clamp_min(1) * t * t


class DistillationModel(BaseModel):
    """``teacher`` and ``student`` are models whose ``predict(input_batch)`` returns a dict with
    ``"logits"`` (or that expose ``compute_logits``); the student must also implement
    ``forward`` returning ``(loss, aux)``.  Mark ``teacher/.*`` with ``UpdateType.NO_UPDATE`` in
    the learner's update rules; gradients never reach it either way."""

    @config_class
    class Config(BaseModel.Config):
        teacher: Required[InstantiableConfig] = REQUIRED
        student: Required[InstantiableConfig] = REQUIRED
        temperature: float = 1.0
        # total = (1 - soft_target_weight) * student loss + soft_target_weight * KL.
        soft_target_weight: float = 0.5
        pad_label: int = -1

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("teacher", cfg.teacher)
        self._add_child("student", cfg.student)

    @staticmethod
    def _logits(model, input_batch: dict) -> Tensor:
        out = model.predict(input_batch)
        if isinstance(out, dict) and "logits" in out:
            return out["logits"]
        return model.compute_logits(out)

    def predict(self, input_batch: dict):
        return self.student.predict(input_batch)

    def forward(self, input_batch: dict):
        cfg = self._config
        with torch.no_grad():
            teacher_logits = self._logits(self.teacher, input_batch)
        student_loss, aux = self.student(input_batch)
        student_logits = aux["logits"] if isinstance(aux, dict) and "logits" in aux else self._logits(self.student, input_batch)
        live = None
        labels = input_batch.get("target_labels", input_batch.get("label"))
        if labels is not None and labels.shape == student_logits.shape[:-1]:
            live = labels != cfg.pad_label
        kl = soft_target_kl(student_logits=student_logits, teacher_logits=teacher_logits.detach(),
                            temperature=cfg.temperature, live=live)
        loss = (1 - cfg.soft_target_weight) * student_loss + cfg.soft_target_weight * kl
        self.add_summary("loss/student", student_loss.detach())
        self.add_summary("loss/soft_target_kl", kl.detach())
        return loss, {"student_logits": student_logits, "teacher_logits": teacher_logits}
