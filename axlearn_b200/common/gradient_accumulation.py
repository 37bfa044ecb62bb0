"""Gradient accumulation over micro-batches as a wrapper around a loss function.

Counterpart of axlearn/common/gradient_accumulation.py (``with_minibatch_steps`` :96-351).  The
trainer has the same behaviour built in (``SpmdTrainer.Config.grad_accumulation_steps``); this is
the stand-alone form for custom loops: the batch is cut into ``steps`` equal slices along dim 0,
every slice runs forward and backward on its own (so activations of one slice are alive at a
time), gradients are summed into ``.grad`` and scaled so that the result equals the gradient of the
mean loss over the whole batch, and scalar outputs are averaged.
"""

from __future__ import annotations

from typing import Any, Callable, Sequence

import torch

from axlearn_b200.common.utils import tree_map

Tensor = torch.Tensor


def split_batch(batch: Any, steps: int) -> list:
    """``steps`` slices of every tensor along dim 0 (all batch dims must be divisible)."""
    def check(t):
        if isinstance(t, Tensor) and t.dim() > 0 and t.shape[0] % steps:
            raise ValueError(f"batch dim {t.shape[0]} is not divisible by {steps} micro-batches")
        return t

    tree_map(check, batch)
    return [tree_map(lambda t: t.chunk(steps, dim=0)[i] if isinstance(t, Tensor) and t.dim() > 0 else t, batch)
            for i in range(steps)]


def with_minibatch_steps(loss_fn: Callable[[Any], tuple[Tensor, dict]], *, steps: int) -> Callable[[Any], tuple[Tensor, dict]]:
    """``loss_fn(batch) -> (mean loss, aux)``.  The returned function also runs the backward passes:
    after it returns, the parameters' ``.grad`` hold the gradient of the whole batch's mean loss."""
    if steps < 1:
        raise ValueError("steps must be positive")

    def wrapped(batch: Any) -> tuple[Tensor, dict]:
        total, aux_sum = None, {}
        for micro in split_batch(batch, steps):
            loss, aux = loss_fn(micro)
            (loss / steps).backward()
            total = loss.detach() / steps if total is None else total + loss.detach() / steps
            for k, v in (aux or {}).items():
                if isinstance(v, Tensor) and v.dim() == 0:
                    aux_sum[k] = aux_sum.get(k, 0) + v.detach() / steps
        return total, aux_sum

    return wrapped
