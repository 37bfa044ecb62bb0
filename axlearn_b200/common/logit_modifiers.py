"""Logits-to-logits functions used while sampling: temperature, top-k, top-p, chains.

Parity targets in the reference (axlearn/common/logit_modifiers.py): ``chain`` (:33),
``scale_by`` (:45), ``top_p_logits`` (:69), ``top_k_logits`` (:124).  The reference finds the
top-k / top-p thresholds with bit-level binary searches because sorting is slow on its
accelerator; a radix sort over the vocabulary is cheap on a GPU, so thresholds here come from
one descending sort per row.
"""

from __future__ import annotations

from typing import Callable, Union

import torch

from axlearn_b200.common.config import maybe_instantiate

Tensor = torch.Tensor
LogitsToLogitsFn = Callable[[Tensor], Tensor]
NEG_INF = -1.0e7


def chain(*args) -> LogitsToLogitsFn:
    """Applies several modifiers (or their configs) in order."""

    def fn(logits: Tensor) -> Tensor:
        for m in args:
            logits = maybe_instantiate(m)(logits)
        return logits

    return fn


def scale_by(temperature: float, *, min_temperature: float = 1e-4) -> LogitsToLogitsFn:
    """``logits / temperature``; refuses temperatures small enough to overflow."""
    if temperature < min_temperature:
        raise ValueError(f"temperature should be >= {min_temperature} for numerical stability.")

    def fn(logits: Tensor) -> Tensor:
        return logits / max(temperature, min_temperature)

    return fn


def top_p_logits(p: Union[float, Tensor]) -> LogitsToLogitsFn:
    """Keeps the smallest set of highest-probability tokens whose mass reaches ``p`` (ties with
    the threshold are all kept); everything else becomes ``NEG_INF``."""
    if not isinstance(p, Tensor) and not 0.0 < p <= 1.0:
        raise ValueError(f"p must be in (0, 1], got {p}")

    def fn(logits: Tensor) -> Tensor:
        probs = torch.softmax(logits.float(), dim=-1)
        sorted_p, _ = probs.sort(dim=-1, descending=True)
        cum = sorted_p.cumsum(dim=-1)
        pp = p if isinstance(p, Tensor) else torch.tensor(p, device=logits.device)
        pp = pp.to(cum.dtype).reshape(pp.shape + (1,) * (cum.dim() - pp.dim())) if pp.dim() else pp
        # First sorted position where the cumulative mass reaches p.
        reached = (cum >= pp - 1e-7).to(torch.int64)
        first = reached.argmax(dim=-1, keepdim=True)
        # Rows where rounding never reaches p keep everything.
        first = torch.where(reached.sum(dim=-1, keepdim=True) > 0, first, torch.full_like(first, logits.shape[-1] - 1))
        threshold = torch.gather(sorted_p, -1, first)
        return torch.where(probs >= threshold, logits, torch.full_like(logits, NEG_INF))

    return fn


def top_k_logits(k: int, *, break_ties: str = "all") -> LogitsToLogitsFn:
    """Keeps the ``k`` largest logits per row.  ``break_ties="all"`` keeps every logit tied with
    the k-th value; ``"smallest_index"`` keeps exactly k, preferring lower indices among ties."""
    if k < 1:
        raise ValueError("k must be >= 1")
    if break_ties not in ("all", "smallest_index"):
        raise NotImplementedError(break_ties)

    def fn(logits: Tensor) -> Tensor:
        kk = min(k, logits.shape[-1])
        neg = torch.full_like(logits, NEG_INF)
        if break_ties == "all":
            kth = logits.topk(kk, dim=-1).values[..., -1:]
            return torch.where(logits >= kth, logits, neg)
        # A stable descending sort orders ties by index.
        order = logits.sort(dim=-1, descending=True, stable=True).indices[..., :kk]
        keep = torch.zeros_like(logits, dtype=torch.bool).scatter_(-1, order, True)
        return torch.where(keep, logits, neg)

    return fn
