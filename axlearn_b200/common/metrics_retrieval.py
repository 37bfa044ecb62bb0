"""Ranking / retrieval metrics over score matrices ``[num_queries, num_items]``.

Parity targets in the reference (axlearn/common/metrics_retrieval.py): ``top_k_accuracy`` (:19),
``top_k_recall`` (:116), ``mean_reciprocal_rank`` (:225), ``average_rank`` (:257),
``average_precision_at_k`` (:295), ``ndcg_at_k`` (:412), ``metric_at_k_name`` (:652).
``relevance_labels`` is ``[num_queries, num_items]`` (> 0 = relevant; graded for nDCG);
``query_padding`` / ``item_paddings`` mask out padded queries / items.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

Tensor = torch.Tensor
_NEG = -1e30


def metric_at_k_name(name: str, k: int) -> str:
    return f"{name}@{k}"


def _masked_scores(sim: Tensor, item_paddings: Optional[Tensor]) -> Tensor:
    sim = sim.float()
    if item_paddings is not None:
        sim = torch.where(item_paddings.bool(), torch.full_like(sim, _NEG), sim)
    return sim


def _ranks(sim: Tensor) -> Tensor:
    """0-based rank of every item in its row, best first (ties broken by index)."""
    order = torch.argsort(sim, dim=-1, descending=True, stable=True)
    ranks = torch.empty_like(order)
    ranks.scatter_(-1, order, torch.arange(sim.shape[-1], device=sim.device).expand_as(order))
    return ranks


def _query_mean(values: Tensor, query_padding: Optional[Tensor]) -> Tensor:
    if query_padding is None:
        return values.mean()
    live = (~query_padding.bool()).float()
    return (values * live).sum() / live.sum().clamp_min(1.0)


def top_k_accuracy(sim: Tensor, *, gt_targets: Optional[Tensor] = None, relevance_labels: Optional[Tensor] = None,
                   top_ks: Sequence[int] = (1,), query_padding: Optional[Tensor] = None,
                   item_paddings: Optional[Tensor] = None) -> list[Tensor]:
    """Share of queries with at least one relevant item among the top k.  ``gt_targets [Q]`` gives
    the single relevant item per query (alternative to ``relevance_labels``)."""
    sim = _masked_scores(sim, item_paddings)
    if relevance_labels is None:
        relevance_labels = torch.zeros_like(sim).scatter_(-1, gt_targets.long()[:, None], 1.0)
    ranks = _ranks(sim)
    rel = relevance_labels > 0
    best = torch.where(rel, ranks, torch.full_like(ranks, sim.shape[-1])).amin(dim=-1)
    return [_query_mean((best < k).float(), query_padding) for k in top_ks]


def top_k_recall(sim: Tensor, *, relevance_labels: Tensor, top_ks: Sequence[int] = (1,),
                 query_padding: Optional[Tensor] = None, item_paddings: Optional[Tensor] = None) -> list[Tensor]:
    """Mean over queries of (relevant items in the top k) / (relevant items)."""
    sim = _masked_scores(sim, item_paddings)
    ranks = _ranks(sim)
    rel = (relevance_labels > 0).float()
    total = rel.sum(dim=-1).clamp_min(1.0)
    return [_query_mean((rel * (ranks < k).float()).sum(dim=-1) / total, query_padding) for k in top_ks]


def mean_reciprocal_rank(sim: Tensor, *, relevance_labels: Tensor, query_padding: Optional[Tensor] = None,
                         item_paddings: Optional[Tensor] = None) -> Tensor:
    sim = _masked_scores(sim, item_paddings)
    ranks = _ranks(sim)
    rel = relevance_labels > 0
    best = torch.where(rel, ranks, torch.full_like(ranks, 10 ** 9)).amin(dim=-1)
    rr = torch.where(rel.any(dim=-1), 1.0 / (best.float() + 1), torch.zeros_like(best, dtype=torch.float32))
    return _query_mean(rr, query_padding)


def average_rank(sim: Tensor, *, relevance_labels: Tensor, query_padding: Optional[Tensor] = None,
                 item_paddings: Optional[Tensor] = None) -> Tensor:
    """Mean 1-based rank of the relevant items."""
    sim = _masked_scores(sim, item_paddings)
    ranks = _ranks(sim).float() + 1
    rel = (relevance_labels > 0).float()
    if query_padding is not None:
        rel = rel * (~query_padding.bool()).float()[:, None]
    return (ranks * rel).sum() / rel.sum().clamp_min(1.0)


def average_precision_at_k(sim: Tensor, *, relevance_labels: Tensor, top_ks: Sequence[int] = (1,),
                           query_padding: Optional[Tensor] = None, item_paddings: Optional[Tensor] = None) -> dict:
    """``{k: AP@k [Q]}``: mean over the relevant items in the top k of precision at their rank,
    normalised by min(k, number of relevant items)."""
    sim = _masked_scores(sim, item_paddings)
    order = torch.argsort(sim, dim=-1, descending=True, stable=True)
    rel_sorted = torch.gather((relevance_labels > 0).float(), -1, order)
    hits = torch.cumsum(rel_sorted, dim=-1)
    positions = torch.arange(1, sim.shape[-1] + 1, device=sim.device).float()
    precision_at = hits / positions
    total = rel_sorted.sum(dim=-1)
    out = {}
    for k in top_ks:
        ap = (precision_at[:, :k] * rel_sorted[:, :k]).sum(dim=-1) / torch.minimum(total, torch.tensor(float(k))).clamp_min(1.0)
        if query_padding is not None:
            ap = torch.where(query_padding.bool(), torch.zeros_like(ap), ap)
        out[k] = ap
    return out


def ndcg_at_k(sim: Tensor, *, relevance_labels: Tensor, top_ks: Sequence[int] = (1,),
              query_padding: Optional[Tensor] = None, item_paddings: Optional[Tensor] = None) -> dict:
    """``{k: mean nDCG@k}`` with gains ``relevance`` and discounts ``1 / log2(rank + 1)``."""
    sim = _masked_scores(sim, item_paddings)
    gains = relevance_labels.float()
    if item_paddings is not None:
        gains = torch.where(item_paddings.bool(), torch.zeros_like(gains), gains)
    order = torch.argsort(sim, dim=-1, descending=True, stable=True)
    ideal = torch.sort(gains, dim=-1, descending=True).values
    got = torch.gather(gains, -1, order)
    discounts = 1.0 / torch.log2(torch.arange(2, sim.shape[-1] + 2, device=sim.device).float())
    out = {}
    for k in top_ks:
        dcg = (got[:, :k] * discounts[:k]).sum(dim=-1)
        idcg = (ideal[:, :k] * discounts[:k]).sum(dim=-1)
        ndcg = torch.where(idcg > 0, dcg / idcg.clamp_min(1e-12), torch.zeros_like(dcg))
        out[k] = _query_mean(ndcg, query_padding)
    return out
