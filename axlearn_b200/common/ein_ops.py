"""``rearrange`` and ``repeat`` with einops-style patterns, on torch tensors.

Counterpart of axlearn/common/ein_ops.py (``rearrange`` :48, ``repeat`` :120): patterns such as
``"b t (n h) -> b n t h"`` or ``"b t d -> b t k d"``.  A pattern compiles once (cached) into a
reshape, a permutation, an optional broadcast and a final reshape, so that calls cost no parsing.
"""

from __future__ import annotations

import functools
import math
import re
from typing import Sequence

import torch

Tensor = torch.Tensor
_TOKEN = re.compile(r"\(|\)|[A-Za-z_][A-Za-z_0-9]*|1|\.\.\.")


def _parse(side: str) -> list[list[str]]:
    """``"b (n h) 1"`` -> ``[["b"], ["n", "h"], []]`` (``1`` is an empty group)."""
    groups: list[list[str]] = []
    cur = None
    for tok in _TOKEN.findall(side):
        if tok == "...":
            raise NotImplementedError("ellipsis is not supported; name the axes")
        if tok == "(":
            if cur is not None:
                raise ValueError(f"nested parentheses in {side!r}")
            cur = []
        elif tok == ")":
            if cur is None:
                raise ValueError(f"unbalanced parentheses in {side!r}")
            groups.append(cur)
            cur = None
        elif tok == "1":
            if cur is None:             # a unit axis of its own; inside a group it changes nothing
                groups.append([])
        else:
            if cur is not None:
                cur.append(tok)
            else:
                groups.append([tok])
    if cur is not None:
        raise ValueError(f"unbalanced parentheses in {side!r}")
    return groups


@functools.lru_cache(maxsize=256)
def _compile(pattern: str):
    if "->" not in pattern:
        raise ValueError(f"pattern needs '->': {pattern!r}")
    lhs, rhs = (s.strip() for s in pattern.split("->"))
    left, right = _parse(lhs), _parse(rhs)
    left_axes = [a for g in left for a in g]
    right_axes = [a for g in right for a in g]
    if len(set(left_axes)) != len(left_axes) or len(set(right_axes)) != len(right_axes):
        raise ValueError(f"an axis name repeats in {pattern!r}")
    return left, right, left_axes, right_axes


def _axis_sizes(x: Tensor, left, sizes: dict) -> dict:
    if x.dim() != len(left):
        raise ValueError(f"tensor of rank {x.dim()} does not match {len(left)} groups")
    known = dict(sizes)
    for dim, group in zip(x.shape, left):
        unknown = [a for a in group if a not in known]
        prod = math.prod(known[a] for a in group if a in known)
        if len(unknown) > 1:
            raise ValueError(f"sizes of {unknown} cannot be inferred; pass them as keyword arguments")
        if unknown:
            if dim % prod:
                raise ValueError(f"dimension {dim} is not divisible by {prod}")
            known[unknown[0]] = dim // prod
        elif prod != dim:
            raise ValueError(f"group {group} has size {prod}, tensor has {dim}")
    return known


def rearrange(x: Tensor, pattern: str, **sizes: int) -> Tensor:
    left, right, left_axes, right_axes = _compile(pattern)
    if set(left_axes) != set(right_axes):
        raise ValueError(f"rearrange keeps the set of axes: {pattern!r}")
    known = _axis_sizes(x, left, sizes)
    y = x.reshape([known[a] for a in left_axes])
    y = y.permute([left_axes.index(a) for a in right_axes])
    return y.reshape([math.prod(known[a] for a in g) for g in right])


def repeat(x: Tensor, pattern: str, **sizes: int) -> Tensor:
    """New axes on the right-hand side are broadcast to the size given by keyword."""
    left, right, left_axes, right_axes = _compile(pattern)
    if not set(left_axes) <= set(right_axes):
        raise ValueError(f"repeat cannot drop axes: {pattern!r}")
    known = _axis_sizes(x, left, sizes)
    new = [a for a in right_axes if a not in left_axes]
    for a in new:
        if a not in known:
            raise ValueError(f"size of the new axis {a!r} is required")
    y = x.reshape([known[a] for a in left_axes] + [1] * len(new))
    order = left_axes + new
    y = y.permute([order.index(a) for a in right_axes])
    y = y.expand([known[a] for a in right_axes])
    return y.reshape([math.prod(known[a] for a in g) for g in right])
