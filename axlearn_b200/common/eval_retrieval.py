"""Retrieval evaluation over embeddings collected from a whole evaluation set.

Reference: axlearn/common/eval_retrieval.py (``calculate_clip_retrieval_metrics`` :111,
``CLIPRetrievalMetricCalculator`` :190, ``EmbeddingRetrievalMetricCalculator`` :259-458,
``KnnMetricCalculator`` :548).  Similarities are computed chunk by chunk over the queries so that
the ``queries x index`` matrix never has to exist in full.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.evaler import GlobalMetricCalculator
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.metrics_retrieval import top_k_accuracy, top_k_recall

Tensor = torch.Tensor


def calculate_clip_retrieval_metrics(*, image_embeddings: Tensor, text_embeddings: Tensor, text_paddings: Tensor,
                                     top_ks: Sequence[int] = (1, 5, 10)) -> dict:
    """``image_embeddings [N, D]``, ``text_embeddings [N, S, D]`` (``S`` captions per image, with
    ``text_paddings [N, S]``).  Text-to-image: every live caption retrieves its image;
    image-to-text: an image counts when any of its captions is in the top k."""
    n, s, d = text_embeddings.shape
    flat_text = text_embeddings.reshape(n * s, d)
    live_text = ~text_paddings.reshape(-1).bool()
    sim_t2i = flat_text @ image_embeddings.t()                              # [N*S, N]
    owner = torch.arange(n, device=sim_t2i.device).repeat_interleave(s)
    out = {}
    t2i = top_k_accuracy(sim_t2i, gt_targets=owner, top_ks=top_ks, query_padding=~live_text)
    relevance = F.one_hot(owner, n).t().float() * live_text[None].float()   # [N, N*S]
    i2t = top_k_accuracy(sim_t2i.t(), relevance_labels=relevance, top_ks=top_ks,
                         item_paddings=(~live_text)[None].expand(n, -1))
    for k, a, b in zip(top_ks, t2i, i2t):
        out[f"text_to_image@{k}"], out[f"image_to_text@{k}"] = a, b
    return out


class CLIPRetrievalMetricCalculator(GlobalMetricCalculator):
    """Expects ``predict`` outputs ``image_embedding [B, D]`` and ``text_embedding [B, D]`` or
    ``[B, S, D]``; optional ``input_batch["text_paddings"] [B, S]``."""

    @config_class
    class Config(GlobalMetricCalculator.Config):
        top_ks: Sequence[int] = (1, 5, 10)
        metric_fn: Optional[object] = None

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        img = torch.cat([o.predict_outputs["image_embedding"].float() for o in all_forward_outputs])
        txt = torch.cat([o.predict_outputs["text_embedding"].float() for o in all_forward_outputs])
        if txt.dim() == 2:
            txt = txt[:, None]
        pads = [o.input_batch.get("text_paddings") for o in all_forward_outputs]
        paddings = torch.cat(pads) if all(p is not None for p in pads) else torch.zeros(txt.shape[:2], dtype=torch.bool)
        metrics = calculate_clip_retrieval_metrics(image_embeddings=img, text_embeddings=txt, text_paddings=paddings,
                                                   top_ks=self._config.top_ks)
        return {self.formatted_metric_name(k): WeightedSummary(v, img.shape[0]) for k, v in metrics.items()}


class EmbeddingRetrievalMetricCalculator(GlobalMetricCalculator):
    """Every example's ``embedding`` queries the index of all examples (itself excluded); items
    with the query's ``label`` are relevant.  Reports recall@k and accuracy@k."""

    @config_class
    class Config(GlobalMetricCalculator.Config):
        top_ks: Sequence[int] = (1, 5)
        embedding_key: str = "embedding"
        label_key: str = "label"
        query_chunk_size: int = 1024
        metric_fn: Optional[object] = None

    def _scores(self, queries: Tensor, index: Tensor) -> Tensor:
        return queries @ index.t()

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        cfg = self._config
        emb = F.normalize(torch.cat([o.predict_outputs[cfg.embedding_key].float() for o in all_forward_outputs]), dim=-1)
        labels = torch.cat([o.input_batch[cfg.label_key] for o in all_forward_outputs])
        n = emb.shape[0]
        sums = {f"accuracy@{k}": 0.0 for k in cfg.top_ks} | {f"recall@{k}": 0.0 for k in cfg.top_ks}
        for lo in range(0, n, cfg.query_chunk_size):
            q = slice(lo, min(n, lo + cfg.query_chunk_size))
            m = q.stop - q.start
            sim = self._scores(emb[q], emb)
            self_mask = torch.zeros(m, n, dtype=torch.bool)
            self_mask[torch.arange(m), torch.arange(q.start, q.stop)] = True
            rel = (labels[q, None] == labels[None, :]).float() * (~self_mask).float()
            acc = top_k_accuracy(sim, relevance_labels=rel, top_ks=cfg.top_ks, item_paddings=self_mask)
            rec = top_k_recall(sim, relevance_labels=rel, top_ks=cfg.top_ks, item_paddings=self_mask)
            for k, a, r in zip(cfg.top_ks, acc, rec):
                sums[f"accuracy@{k}"] += float(a) * m
                sums[f"recall@{k}"] += float(r) * m
        return {self.formatted_metric_name(k): WeightedSummary(torch.tensor(v / max(n, 1)), n) for k, v in sums.items()}


class KnnMetricCalculator(EmbeddingRetrievalMetricCalculator):
    """k-nearest-neighbour classification accuracy: the majority label among the top k."""

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        cfg = self._config
        emb = F.normalize(torch.cat([o.predict_outputs[cfg.embedding_key].float() for o in all_forward_outputs]), dim=-1)
        labels = torch.cat([o.input_batch[cfg.label_key] for o in all_forward_outputs]).long()
        n = emb.shape[0]
        sim = emb @ emb.t()
        sim.fill_diagonal_(-1e9)
        out = {}
        for k in cfg.top_ks:
            nn_labels = labels[sim.topk(min(k, n - 1), dim=-1).indices]
            votes = F.one_hot(nn_labels, int(labels.max()) + 1).sum(dim=1)
            out[self.formatted_metric_name(f"knn_accuracy@{k}")] = WeightedSummary(
                (votes.argmax(-1) == labels).float().mean(), n)
        return out
