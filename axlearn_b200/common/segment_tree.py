"""Segment trees for best-fit sequence packing.

Counterpart of axlearn/common/segment_tree.py (``SegmentTree`` :13, ``BestFitSegmentTree`` :151).
Best-fit packing keeps, for every remaining capacity ``0..max_len``, how many open bins have it,
and asks for the smallest capacity ``>= length`` in ``O(log max_len)``: a max-tree over capacities
finds it by descending towards the leftmost leaf that can hold the item.
"""

from __future__ import annotations

from typing import Callable, Generic, Optional, Sequence, TypeVar

T = TypeVar("T")


class SegmentTree(Generic[T]):
    """Array of ``n`` values with point updates and ``reduce(lo, hi)`` over ``[lo, hi)`` for an
    associative ``op`` with identity ``identity``."""

    def __init__(self, n: int, op: Callable[[T, T], T], identity: T, values: Optional[Sequence[T]] = None):
        self._n, self._op, self._id = n, op, identity
        self._size = 1
        while self._size < max(1, n):
            self._size *= 2
        self._tree = [identity] * (2 * self._size)
        if values is not None:
            for i, v in enumerate(values):
                self._tree[self._size + i] = v
            for i in range(self._size - 1, 0, -1):
                self._tree[i] = op(self._tree[2 * i], self._tree[2 * i + 1])

    def __len__(self):
        return self._n

    def __getitem__(self, i: int) -> T:
        return self._tree[self._size + i]

    def update(self, i: int, value: T) -> None:
        if not 0 <= i < self._n:
            raise IndexError(i)
        i += self._size
        self._tree[i] = value
        i //= 2
        while i:
            self._tree[i] = self._op(self._tree[2 * i], self._tree[2 * i + 1])
            i //= 2

    def reduce(self, lo: int = 0, hi: Optional[int] = None) -> T:
        hi = self._n if hi is None else hi
        left, right = self._id, self._id
        lo += self._size
        hi += self._size
        while lo < hi:
            if lo & 1:
                left = self._op(left, self._tree[lo])
                lo += 1
            if hi & 1:
                hi -= 1
                right = self._op(self._tree[hi], right)
            lo //= 2
            hi //= 2
        return self._op(left, right)

    def leftmost(self, lo: int, predicate: Callable[[T], bool]) -> int:
        """The smallest ``i >= lo`` with ``predicate(value_i)``, assuming ``predicate`` of a
        reduction holds iff it holds for one of its elements (e.g. ``max >= x``); -1 if none."""
        for i in self._descend(1, 0, self._size, lo, predicate):
            return i
        return -1

    def _descend(self, node, node_lo, node_hi, lo, predicate):
        if node_hi <= lo or not predicate(self._tree[node]):
            return
        if node >= self._size:
            if node_lo < self._n:
                yield node_lo
            return
        mid = (node_lo + node_hi) // 2
        yield from self._descend(2 * node, node_lo, mid, lo, predicate)
        yield from self._descend(2 * node + 1, mid, node_hi, lo, predicate)


class BestFitSegmentTree:
    """Open bins by remaining capacity; ``best_fit(length)`` returns the tightest capacity that
    holds ``length`` (an empty bin of capacity ``max_len`` is always available)."""

    def __init__(self, max_len: int):
        self._max = max_len
        self._count = [0] * (max_len + 1)
        # Leaf c holds c when some open bin has remaining capacity c, else -1.
        self._tree: SegmentTree[int] = SegmentTree(max_len + 1, max, -1, values=[-1] * max_len + [max_len])

    def best_fit(self, length: int) -> int:
        if not 0 < length <= self._max:
            raise ValueError(f"length {length} outside (0, {self._max}]")
        return self._tree.leftmost(length, lambda m: m >= length)

    def place(self, length: int) -> tuple[int, int]:
        """Puts an item into its best-fitting bin; returns ``(capacity before, capacity after)``."""
        cap = self.best_fit(length)
        if cap != self._max:                        # the fresh bin never runs out
            self._count[cap] -= 1
            if self._count[cap] == 0:
                self._tree.update(cap, -1)
        rest = cap - length
        if rest > 0:
            self._count[rest] += 1
            self._tree.update(rest, rest)
        return cap, rest


def best_fit_pack(lengths: Sequence[int], max_len: int) -> list[list[int]]:
    """Bins of item indices: every item goes to the open bin with the least room that still holds
    it (first opened among equals), or to a new bin."""
    tree = BestFitSegmentTree(max_len)
    by_capacity: dict[int, list[int]] = {}
    bins: list[list[int]] = []
    for i, n in enumerate(lengths):
        n = min(n, max_len)
        cap, rest = tree.place(n)
        if cap == max_len and not by_capacity.get(cap):
            bins.append([])
            b = len(bins) - 1
        else:
            b = by_capacity[cap].pop(0)
        bins[b].append(i)
        if rest > 0:
            by_capacity.setdefault(rest, []).append(b)
    return bins
