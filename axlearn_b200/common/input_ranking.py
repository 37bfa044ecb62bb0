"""Ranking-task input processing.

Parity target: axlearn/common/input_ranking.py:11 ``rank_by_value``.
"""

from __future__ import annotations

import numpy as np

from axlearn_b200.common.input_processing import DatasetToDatasetFn, Example, map_over_dataset


def rank_by_value(*, input_key: str, output_key: str, ascending: bool, allow_ties: bool) -> DatasetToDatasetFn:
    """Stores the 1-based rank of every element of the rank-1 ``input_key`` in ``output_key``.
    ``allow_ties``: equal values share the lowest of their ranks and leave gaps after
    (``[2, 2, 4] -> [1, 1, 3]``); otherwise a stable sort breaks ties by position (``[1, 2, 3]``)."""

    def fn(ex: Example) -> Example:
        values = np.asarray(ex[input_key])
        if values.ndim != 1:
            raise NotImplementedError(f"Only implemented for rank-1 tensors. Got rank-{values.ndim}.")
        keyed = values if ascending else -values
        order = np.argsort(keyed, kind="stable")
        ranks = np.empty_like(order)
        ranks[order] = np.arange(len(order))
        if allow_ties:
            sorted_vals = keyed[order]
            # First sorted position of each run of equal values.
            first = np.concatenate([[0], np.flatnonzero(sorted_vals[1:] != sorted_vals[:-1]) + 1]) if len(order) else order
            run = np.cumsum(np.concatenate([[0], (sorted_vals[1:] != sorted_vals[:-1]).astype(np.int64)])) if len(order) else order
            ranks = first[run][ranks]
        ex = dict(ex)
        ex[output_key] = (ranks + 1).astype(np.int32)
        return ex

    return map_over_dataset(fn)
