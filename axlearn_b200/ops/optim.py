"""Multi-tensor optimizer steps.

``multi_tensor_adamw`` applies, for every listed tensor, in one pass over memory::

    g' = grad_scale * g                         (global-norm clip folded in)
    m  = b1*m + (1-b1)*g' ;  v = b2*v + (1-b2)*g'^2
    p -= lr * (m/(1-b1^t)) / (sqrt(v/(1-b2^t)) + eps) + weight_decay * wd_scale * p
    shadow = cast(p)                            (low-precision copy read by the model)

which is the closed form of the reference's chains ``adamw_optimizer`` /
``adamw_decoupled_optimizer`` (axlearn/common/optimizers.py:741-856) with ``lr`` and
``weight_decay`` already multiplied by the schedules for this step.  On GPU all tensors are
processed by a single launch of the sm_100a kernel (pointer table + chunk table); on CPU the
same arithmetic runs per tensor in PyTorch.
"""

from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

from axlearn_b200.ops import dispatch, reference


def multi_tensor_adamw(
    *,
    params: Sequence[torch.Tensor],
    grads: Sequence[torch.Tensor],
    mus: Sequence[torch.Tensor],
    nus: Sequence[torch.Tensor],
    shadows: Sequence[Optional[torch.Tensor]],
    wd_scales: Sequence[float],
    step: int,
    lr: float,
    weight_decay: float,
    b1: float,
    b2: float,
    eps: float,
    grad_scale: Union[float, torch.Tensor] = 1.0,
) -> None:
    if not params:
        return
    on_gpu = all(p.is_cuda for p in params) and not dispatch._flags.force_reference  # pylint: disable=protected-access
    if on_gpu and all(p.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32
                      for p, m, v in zip(params, mus, nus)):
        dispatch._ops().multi_tensor_adamw(  # pylint: disable=protected-access
            params, grads, mus, nus, shadows, wd_scales, step=step, lr=lr, weight_decay=weight_decay,
            b1=b1, b2=b2, eps=eps, grad_scale=grad_scale)
        return
    gs = grad_scale
    for p, g, m, v, sh, ws in zip(params, grads, mus, nus, shadows, wd_scales):
        scale = gs.to(p.device) if isinstance(gs, torch.Tensor) else gs
        reference.adamw_step(
            p, g, m, v, step=step, lr=lr, b1=b1, b2=b2, eps=eps, weight_decay=weight_decay * ws,
            update_scale=1.0, grad_scale=scale)
        if sh is not None and sh is not p:
            sh.copy_(p)
