"""Attention kernels: flash forward/backward for training and prefill, KV-cache append.

``flash_attention`` takes ``q [B, T, N, H]``, ``k/v [B, S, Nkv, H]`` (bf16) and returns
``[B, T, N, H]``; GQA is handled by head grouping inside the kernel (K/V are never repeated in
memory).  The forward also produces the per-row log-sum-exp which the backward consumes.

Reference behaviour being replaced: the Pallas-Triton kernels
(axlearn/common/flash_attention/gpu_attention.py:114-243 forward, :436-616 backward) and the
cuDNN fused attention the reference prefers on GPU (:792-926).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from axlearn_b200.ops import cuda_ops


def _has(symbol: str) -> bool:
    return hasattr(cuda_ops.lib(), symbol)


def flash_supported(q, k, v, segment_ids=None) -> bool:
    """Head dims 64 / 128 with grouped KV heads; causal, segment-id, sliding-window and
    logit-cap masks all run inside the kernels."""
    h = q.shape[-1]
    if segment_ids is not None and (segment_ids.dim() != 2 or segment_ids.shape[1] != q.shape[1]):
        return False
    return h in (64, 128) and q.shape[2] % k.shape[2] == 0


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, q_seg, k_seg, window, logit_cap):
        from axlearn_b200.common import remat
        from axlearn_b200.ops import flash_sm100

        def run():
            ranges = flash_sm100.segment_tile_ranges(q_seg, k_seg) if q_seg is not None else None
            return flash_sm100.forward(q, k, v, causal=causal, scale=scale, q_seg=q_seg, k_seg=k_seg,
                                       ranges=ranges, window=window, logit_cap=logit_cap)

        # Under a remat policy that keeps the context, the first pass stores (out, lse) and the
        # replay finds them here instead of launching the forward kernel again.
        (out, lse), replayed = remat.operator_outputs(run, is_dot=False)
        if replayed:
            out = out.view_as(out)
        ctx.save_for_backward(q, k, v, out, lse, q_seg, k_seg)
        ctx.causal, ctx.scale, ctx.window, ctx.logit_cap = causal, scale, window, logit_cap
        ctx.bwd_variant = flash_sm100.BACKWARD_VARIANT  # the selection in force when the forward ran
        return out

    @staticmethod
    def backward(ctx, dout):
        from axlearn_b200.ops import flash_sm100

        q, k, v, out, lse, q_seg, k_seg = ctx.saved_tensors
        k_ranges = flash_sm100.segment_tile_ranges(k_seg, q_seg) if q_seg is not None else None
        dq, dk, dv = flash_sm100.backward(
            q, k, v, out, lse, dout.contiguous(), causal=ctx.causal, scale=ctx.scale, q_seg=q_seg, k_seg=k_seg,
            k_ranges=k_ranges, window=ctx.window, logit_cap=ctx.logit_cap, variant=ctx.bwd_variant)
        return dq, dk, dv, None, None, None, None, None, None


def flash_attention(q, k, v, *, causal: bool, softmax_scale: Optional[float], segment_ids=None,
                    kv_segment_ids=None, sliding_window: Optional[int] = None, logit_cap: Optional[float] = None):
    """``segment_ids [B, T]`` (and ``kv_segment_ids [B, S]``, default the same tensor): a query
    sees only keys of its own segment.  ``sliding_window``: keys more than that many positions
    before the query are hidden.  ``logit_cap``: scaled scores become ``cap * tanh(s / cap)``."""
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    q_seg = k_seg = None
    if segment_ids is not None:
        q_seg = segment_ids.to(torch.int32).contiguous()
        k_seg = q_seg if kv_segment_ids is None else kv_segment_ids.to(torch.int32).contiguous()
        if k_seg.shape[1] != k.shape[1]:
            raise ValueError("kv_segment_ids must be given when the key length differs from the query length")
    return _FlashAttention.apply(
        q.contiguous(), k.contiguous(), v.contiguous(), bool(causal), float(scale), q_seg, k_seg,
        None if sliding_window is None else int(sliding_window), None if not logit_cap else float(logit_cap))


def paged_kv_append(pages: torch.Tensor, new: torch.Tensor, page_ids: torch.Tensor, offsets: torch.Tensor):
    """In place: ``pages[page_ids[b, s], offsets[b, s]] = new[b, s]``; returns ``pages``."""
    if _has("axb_paged_kv_append"):
        b, s = new.shape[:2]
        row = new.shape[2] * new.shape[3]
        new_c = new.to(pages.dtype).contiguous()
        pid = page_ids.to(torch.int32).contiguous()
        off = offsets.to(torch.int32).contiguous()
        cuda_ops._check(cuda_ops.lib().axb_paged_kv_append(  # pylint: disable=protected-access
            pages.data_ptr(), new_c.data_ptr(), pid.data_ptr(), off.data_ptr(), b * s, row,
            pages.shape[1], cuda_ops._stream()), "axb_paged_kv_append")  # pylint: disable=protected-access
        return pages
    return pages.index_put_((page_ids, offsets), new.to(pages.dtype))
