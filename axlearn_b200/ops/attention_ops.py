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


def flash_supported(q, k, v, segment_ids) -> bool:
    h = q.shape[-1]
    return h in (64, 128) and q.shape[2] % k.shape[2] == 0 and segment_ids is None


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        from axlearn_b200.ops import flash_sm100

        out, lse = flash_sm100.forward(q, k, v, causal=causal, scale=scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        from axlearn_b200.ops import flash_sm100

        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = flash_sm100.backward(q, k, v, out, lse, dout.contiguous(), causal=ctx.causal, scale=ctx.scale)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, *, causal: bool, softmax_scale: Optional[float], segment_ids=None):
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _FlashAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), bool(causal), float(scale))


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
