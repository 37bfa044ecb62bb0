"""Backend selection for the hot ops.

Rule: CUDA tensors in bf16 (fp32 where a kernel supports it) go to the sm_100a kernels in
``axlearn_b200.ops.cuda_ops``; everything else runs the PyTorch statements in
``axlearn_b200.ops.reference``.  ``use_reference_ops()`` forces the reference path (tests
use it to produce oracles on the GPU).
"""

from __future__ import annotations

import contextlib
import threading
from typing import Optional

import torch

from axlearn_b200.ops import reference


class _Flags(threading.local):
    force_reference = 0


_flags = _Flags()


@contextlib.contextmanager
def use_reference_ops():
    _flags.force_reference += 1
    try:
        yield
    finally:
        _flags.force_reference -= 1


def _cuda(*tensors: torch.Tensor) -> bool:
    if _flags.force_reference:
        return False
    return all(t is None or t.is_cuda for t in tensors) and any(t is not None for t in tensors)


def _ops():
    from axlearn_b200.ops import cuda_ops

    return cuda_ops


def rms_norm(x, scale, eps: float, *, upcast: bool = False):
    if _cuda(x, scale) and x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] % 8 == 0:
        return _ops().rms_norm(x, scale, eps)
    return reference.rms_norm(x, scale, eps, upcast=upcast)


def _fused_norm_ok(x, scale) -> bool:
    return _cuda(x, scale) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


def rms_norm_keep_input(x, scale, eps: float, *, upcast: bool = False):
    """``(rms_norm(x), x)``: on the kernel path the gradient that arrives through the second
    output (the residual branch of a pre-norm block) is added inside the norm's backward kernel."""
    if _fused_norm_ok(x, scale):
        return _ops().rms_norm_keep_input(x, scale, eps)
    return rms_norm(x, scale, eps, upcast=upcast), x


def add_rms_norm(x, r, scale, eps: float, *, upcast: bool = False):
    """``(x + r, rms_norm(x + r))``; one pass forward and one backward on the kernel path."""
    if _fused_norm_ok(x, scale) and r.dtype == x.dtype and r.shape == x.shape:
        return _ops().add_rms_norm(x, r, scale, eps)
    total = x + r
    return total, rms_norm(total, scale, eps, upcast=upcast)


def share_input_grad(x):
    """Marks ``x`` as the common input of several linears whose input gradients the kernels then
    sum in the GEMM epilogue (no add kernels); identity elsewhere.  Use only where ``x`` feeds
    nothing but those linears."""
    if _cuda(x) and x.dtype == torch.bfloat16 and x.requires_grad:
        return _ops().share_input_grad(x)
    return x


def swiglu(gate, up):
    if _cuda(gate, up) and gate.dtype == torch.bfloat16:
        return _ops().swiglu(gate, up)
    return reference.swiglu(gate, up)


def rope(x, positions, theta: float = 10000.0):
    if _cuda(x) and x.dtype == torch.bfloat16 and positions.dim() == 1:
        return _ops().rope(x, positions, theta)
    return reference.rope(x, positions, theta)


class _LinearKept(torch.autograd.Function):
    """``x @ w`` whose forward result was kept from the first pass of a replayed layer: nothing
    is computed in forward, and the backward of a matrix product never needs its result."""

    @staticmethod
    def forward(ctx, x, w, y):
        ctx.save_for_backward(x, w)
        return y.view_as(y)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.matmul(dy, w.t())
        if ctx.needs_input_grad[1]:
            dw = torch.matmul(x.reshape(-1, x.shape[-1]).t(), dy.reshape(-1, dy.shape[-1]))
        return dx, dw, None


def _linear_impl(x, w):
    if _cuda(x, w) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        return _ops().linear(x, w)
    return torch.matmul(x, w)


def linear(x, w):
    """``x[..., K] @ w[K, N]`` with fp32 accumulation.  Inside a replayed layer whose remat
    policy keeps this product (``axlearn_b200.common.remat``), the replay reuses the kept result
    instead of running the GEMM again."""
    from axlearn_b200.common import remat

    if remat.active() is None:
        return _linear_impl(x, w)
    on_kernel = _cuda(x, w) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    # A GEMM that carries a parameter gather for a neighbouring layer has to run even when its
    # own result is known.
    can_skip = not (on_kernel and _ops().carries_gather(w))
    (y,), replayed = remat.operator_outputs(lambda: (_linear_impl(x, w),), is_dot=True, can_skip=can_skip)
    if not replayed:
        return y
    if on_kernel:
        return _ops().linear_kept(x, w, y)
    return _LinearKept.apply(x, w, y)


def attention(
    q,
    k,
    v,
    *,
    bias=None,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    segment_ids=None,
    kv_segment_ids=None,
    sliding_window: Optional[int] = None,
    logit_cap: Optional[float] = None,
    dropout_mask=None,
    q_offset: Optional[int] = None,
):
    """``q_offset``: position of the first query among the keys; only ``len(keys) - len(queries)``
    (queries are the last positions: decoding, context parallelism) or None / 0 with equal lengths
    are supported."""
    if q_offset is not None and q_offset != k.shape[1] - q.shape[1]:
        raise NotImplementedError("q_offset must equal len(keys) - len(queries)")
    if (
        _cuda(q, k, v)
        and q.dtype == torch.bfloat16
        and bias is None
        and dropout_mask is None
        and (segment_ids is None or q.shape[1] == k.shape[1] or kv_segment_ids is not None)
        and _ops().flash_supported(q, k, v, segment_ids)
    ):
        # Segment ids, the sliding window and the logit cap are masks of the kernel itself; only an
        # arbitrary additive bias or a dropout mask needs the materialised [T, S] path below.
        # (Under a remat policy that keeps the context, the replay skips the forward kernel.)
        return _ops().flash_attention(
            q, k, v, causal=causal, softmax_scale=softmax_scale, segment_ids=segment_ids,
            kv_segment_ids=kv_segment_ids, sliding_window=sliding_window, logit_cap=logit_cap
        )
    return reference.attention(
        q,
        k,
        v,
        bias=bias,
        causal=causal,
        softmax_scale=softmax_scale,
        segment_ids=segment_ids,
        kv_segment_ids=kv_segment_ids,
        sliding_window=sliding_window,
        logit_cap=logit_cap,
        dropout_mask=dropout_mask,
        q_offset=(None if not q_offset else torch.full((q.shape[0],), q_offset, device=q.device)),
    )


def cross_entropy(logits, targets, *, live_targets=None, z_loss_scale: float = 0.0, denominator=None):
    if _cuda(logits) and logits.dtype in (torch.bfloat16, torch.float32) and logits.dim() >= 2:
        return _ops().cross_entropy(
            logits, targets, live_targets=live_targets, z_loss_scale=z_loss_scale, denominator=denominator
        )
    return reference.cross_entropy(
        logits, targets, live_targets=live_targets, z_loss_scale=z_loss_scale, denominator=denominator
    )


def lm_head_cross_entropy(
    hidden,
    weight,
    targets,
    *,
    live_targets=None,
    z_loss_scale: float = 0.0,
    denominator=None,
    chunk_tokens: int = 8192,
    weight_is_vocab_major: bool = True,
):
    """Fused LM head + cross entropy over token chunks: logits ``[chunk, V]`` exist only for
    one chunk at a time, in forward and in backward (the analogue of the reference's
    ``scan_chunk`` at axlearn/common/causal_lm.py:637-806).

    hidden: [..., D]; weight: [V, D] (vocab-major) or [D, V]; targets: [...].
    Returns ``(loss, aux)`` like ``cross_entropy``.
    """
    from axlearn_b200.ops.chunked_ce import chunked_lm_head_cross_entropy

    return chunked_lm_head_cross_entropy(
        hidden,
        weight,
        targets,
        live_targets=live_targets,
        z_loss_scale=z_loss_scale,
        denominator=denominator,
        chunk_tokens=chunk_tokens,
        weight_is_vocab_major=weight_is_vocab_major,
    )
