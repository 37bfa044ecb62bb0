"""Retrieval metrics of a text dual encoder: accuracy@k, rank of the first hit, nDCG@k.

Reference: axlearn/common/metrics_text_dual_encoder.py (:28 metrics from embeddings, :83 metrics
from the similarity matrix, :176 ``TextDualEncoderMetricCalculator``).  Retrieval is asymmetric:
every live query ranks all keys of the evaluation set (all positives, then all negatives);
padded keys are masked out; the relevant keys of query ``i`` are its own live positives.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.evaler import GlobalMetricCalculator
from axlearn_b200.common.loss import contrastive_logits
from axlearn_b200.common.metrics_retrieval import _masked_scores, _query_mean, _ranks, ndcg_at_k
from axlearn_b200.common.text_dual_encoder import (
    FLATTENED_LEFT_EMBEDDINGS,
    FLATTENED_RIGHT_EMBEDDINGS,
    NEGATIVE_EMBEDDINGS,
    NEGATIVE_PADDINGS,
    POSITIVE_EMBEDDINGS,
    POSITIVE_PADDINGS,
    RIGHT_PADDINGS,
    flatten_and_concat_embeddings,
)

Tensor = torch.Tensor


def calculate_retrieval_metrics_from_similarity_matrix(
        *, sim: Tensor, text_positive_paddings: Tensor, query_paddings: Tensor, text_paddings: Tensor,
        top_ks_for_accuracy: Sequence[int], top_ks_for_ndcg: Optional[Sequence[int]] = None) -> dict:
    """``sim [queries, queries * (positives + negatives)]``; ``text_positive_paddings [queries,
    positives]``; ``query_paddings [queries, 1]``; ``text_paddings`` over the keys."""
    n, p = text_positive_paddings.shape
    relevance = torch.zeros_like(sim, dtype=torch.float32)
    own = torch.arange(n * p, device=sim.device).reshape(n, p)
    relevance.scatter_(1, own, (1 - text_positive_paddings.float()))
    relevance = relevance * (1 - text_paddings.float())[None, :]
    masked = _masked_scores(sim, text_paddings.bool()[None, :].expand_as(sim))
    ranks = _ranks(masked)
    has_hit = relevance.sum(-1) > 0
    first = torch.where(relevance > 0, ranks, torch.full_like(ranks, sim.shape[-1])).amin(-1)
    q_pad = query_paddings.reshape(-1).bool()
    metrics = {}
    for k in top_ks_for_accuracy:
        metrics[f"retrieval_accuracy@{k}"] = _query_mean(((first < k) & has_hit).float(), q_pad)
    metrics["avg_rank"] = _query_mean(torch.where(has_hit, first.float() + 1, torch.zeros(())), q_pad)
    if top_ks_for_ndcg:
        # Queries without any live relevant key do not count.
        ndcg = ndcg_at_k(masked, relevance_labels=relevance, top_ks=top_ks_for_ndcg,
                         query_padding=q_pad | ~has_hit)
        for k in top_ks_for_ndcg:
            metrics[f"ndcg@{k}"] = ndcg[k]
    return metrics


def calculate_retrieval_metrics_from_embeddings(
        *, top_ks_for_accuracy: Sequence[int], query_embeddings: Tensor, query_paddings: Tensor,
        text_positive_embeddings: Tensor, text_positive_paddings: Tensor,
        text_negative_embeddings: Optional[Tensor] = None, text_negative_paddings: Optional[Tensor] = None,
        top_ks_for_ndcg: Optional[Sequence[int]] = None) -> dict:
    flat = flatten_and_concat_embeddings(
        left_positive_embeddings=query_embeddings, right_positive_embeddings=text_positive_embeddings,
        right_positive_paddings=text_positive_paddings, right_negative_embeddings=text_negative_embeddings,
        right_negative_paddings=text_negative_paddings)
    sim = contrastive_logits(flat[FLATTENED_LEFT_EMBEDDINGS], flat[FLATTENED_RIGHT_EMBEDDINGS])
    return calculate_retrieval_metrics_from_similarity_matrix(
        sim=sim, text_positive_paddings=text_positive_paddings, query_paddings=query_paddings,
        text_paddings=flat[RIGHT_PADDINGS], top_ks_for_accuracy=top_ks_for_accuracy,
        top_ks_for_ndcg=top_ks_for_ndcg)


class TextDualEncoderMetricCalculator(GlobalMetricCalculator):
    """Collects every eval batch's embeddings and ranks all keys of the set per query."""

    @config_class
    class Config(GlobalMetricCalculator.Config):
        left_encoder_name: Required[str] = REQUIRED
        right_encoder_name: Required[str] = REQUIRED
        top_ks_for_accuracy: Required[Sequence[int]] = REQUIRED
        top_ks_for_ndcg: Optional[Sequence[int]] = None
        metric_fn: Optional[object] = None            # computed here, not by a callback

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        from axlearn_b200.common.metrics import WeightedSummary

        cfg = self._config

        def cat(get):
            vals = [get(o) for o in all_forward_outputs]
            return None if any(v is None for v in vals) else torch.cat(vals, dim=0)

        left, right = cfg.left_encoder_name, cfg.right_encoder_name
        neg = cat(lambda o: o.predict_outputs[right].get(NEGATIVE_EMBEDDINGS))
        metrics = calculate_retrieval_metrics_from_embeddings(
            top_ks_for_accuracy=cfg.top_ks_for_accuracy, top_ks_for_ndcg=cfg.top_ks_for_ndcg,
            query_embeddings=cat(lambda o: o.predict_outputs[left][POSITIVE_EMBEDDINGS]),
            query_paddings=cat(lambda o: o.input_batch[left][POSITIVE_PADDINGS]),
            text_positive_embeddings=cat(lambda o: o.predict_outputs[right][POSITIVE_EMBEDDINGS]),
            text_positive_paddings=cat(lambda o: o.input_batch[right][POSITIVE_PADDINGS]),
            text_negative_embeddings=neg,
            text_negative_paddings=None if neg is None else cat(lambda o: o.input_batch[right][NEGATIVE_PADDINGS]))
        return {k: WeightedSummary(torch.as_tensor(v), 1) for k, v in metrics.items()}
