"""Python entry points of the decode-time kernels (``csrc/decode_attn.cu``, ``csrc/peer_sync.cu``).

* ``paged_decode_attention``: one query token per sequence over a paged KV cache.
* ``rope_append_paged``: RoPE on q/k of the new token + store of k/v into its page slot.
* ``swiglu_packed``: SwiGLU on a ``[rows, 2F]`` (gate | up) GEMM output.
* ``OneShotAllReduce``: push-based all-reduce over peer memory for latency-bound messages.

A torch reference of the attention (``reference_paged_attention``) is the oracle in tests; it
gathers the pages like the reference's ``PagedKVCache`` does
(axlearn/common/kv_cache/paged_kv_cache.py:22-35).
"""

from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from axlearn_b200.ops import cuda_ops

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
_configured = False


def _lib():
    global _configured
    h = cuda_ops.lib()
    if not _configured:
        h.axb_decode_attn_scratch_floats.argtypes = [c_int, c_int, c_int]
        h.axb_decode_attn_scratch_floats.restype = c_int64
        h.axb_decode_attn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
        h.axb_decode_attn.restype = c_int
        h.axb_rope_append_paged.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                            c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
        h.axb_rope_append_paged.restype = c_int
        h.axb_swiglu_packed.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_void_p]
        h.axb_swiglu_packed.restype = c_int
        h.axb_allreduce_push.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                         c_int64, c_void_p]
        h.axb_allreduce_push.restype = c_int
        h.axb_allreduce_finish.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64,
                                           c_void_p, c_void_p]
        h.axb_allreduce_finish.restype = c_int
        _configured = True
    return h


def _kernel_shape(batch: int, num_kv_heads: int, group: int) -> tuple[int, int]:
    """``(CTAs of one split, CTAs that fit one SM)`` of the kernel that the launcher picks (mirrors
    ``axb_decode_attn``): 128 threads each, residency limited by registers -- 64 with the occupancy
    bound / 125 / 193 for the per-head kernel with 1 / 2 / 4 query heads per CTA, 225 for the
    row-contiguous kernel of four KV heads x four query heads."""
    mode = os.environ.get("AXB_DECODE_ATTN", "")
    natural = 4 if group % 4 == 0 else 2 if group % 2 == 0 else 1
    if mode.startswith("head"):
        gt = min(natural, {"head1": 1, "head2": 2}.get(mode, 4))
    elif group == 4 and num_kv_heads % 4 == 0 and batch * (num_kv_heads // 4) > 8:
        return batch * (num_kv_heads // 4), 2
    else:
        gt = 1 if group == 2 or (group == 4 and num_kv_heads % 4 == 0) else natural
    return batch * num_kv_heads * (group // gt), {1: 8, 2: 4, 4: 2}[gt]


def default_splits(batch: int, num_kv_heads: int, group: int, max_len: int, page_size: int, sms: int = 148) -> int:
    """KV splits: enough CTAs for up to four per SM without splitting below 8 pages; once that grid
    is more than one wave of resident CTAs, the nearby split count whose last wave is fullest (the
    CTAs of a decode step all run about equally long, so a grid of 1.15 waves takes the time of 2)."""
    ctas, resident = _kernel_shape(batch, num_kv_heads, group)
    pages = max(1, max_len // page_size)
    smax = max(1, min(pages // 8 if pages >= 8 else 1, 32))
    base = max(1, min((min(4, resident) * sms + ctas - 1) // ctas, smax))
    slots = sms * resident
    if ctas * base <= slots:
        return base

    def fill(s: int) -> float:
        x = ctas * s / slots
        return x / math.ceil(x)

    candidates = range(max(1, base - 4), min(smax, base + 7) + 1)
    best = max(fill(s) for s in candidates)
    return next(s for s in candidates if fill(s) >= 0.95 * best)


def paged_decode_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                           lengths: torch.Tensor, *, softmax_scale: Optional[float] = None, splits: int = 1,
                           out: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q ``[B, Nq, H]``; pools ``[num_pages, page_size, Nkv, H]``; page_table ``[B, max_pages]`` int32;
    lengths ``[B]`` int32 (valid tokens per sequence).  Returns ``[B, Nq, H]``."""
    b, nq, h = q.shape
    _, page_size, nkv, _ = k_pool.shape
    assert q.is_contiguous() and k_pool.is_contiguous() and v_pool.is_contiguous()
    assert page_table.dtype == torch.int32 and lengths.dtype == torch.int32 and page_table.is_contiguous()
    if out is None:
        out = torch.empty_like(q)
    if splits > 1 and scratch is None:
        scratch = torch.empty(_lib().axb_decode_attn_scratch_floats(b, nq, splits), dtype=torch.float32, device=q.device)
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(h)
    rc = _lib().axb_decode_attn(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(),
                                lengths.data_ptr(), out.data_ptr(), None if scratch is None else scratch.data_ptr(),
                                b, nq, nkv, h, page_size, page_table.shape[1], splits, scale,
                                cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_decode_attn")  # pylint: disable=protected-access
    return out


def reference_paged_attention(q, k_pool, v_pool, page_table, lengths, *, softmax_scale=None):
    """fp32 torch oracle: gather each sequence's pages, mask beyond its length, softmax, PV."""
    b, nq, h = q.shape
    _, page_size, nkv, _ = k_pool.shape
    g = nq // nkv
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(h)
    k = k_pool[page_table.long()].reshape(b, -1, nkv, h).float()
    v = v_pool[page_table.long()].reshape(b, -1, nkv, h).float()
    qf = q.float().reshape(b, nkv, g, h)
    logits = torch.einsum("bkgh,bskh->bkgs", qf, k) * scale
    mask = torch.arange(k.shape[1], device=q.device)[None] < lengths[:, None]
    logits = logits.masked_fill(~mask[:, None, None, :], float("-inf"))
    p = torch.softmax(logits, dim=-1)
    return torch.einsum("bkgs,bskh->bkgh", p, v).reshape(b, nq, h)


def rope_append_paged(qkv: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                      lengths: torch.Tensor, *, num_q_heads: int, theta: float, apply_rope: bool = True,
                      q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """qkv ``[B, (Nq + 2 Nkv) * H]`` of the token at position ``lengths - 1``: returns rotated q
    ``[B, Nq, H]`` and stores rotated k / plain v into the pools."""
    b = qkv.shape[0]
    _, page_size, nkv, h = k_pool.shape
    assert qkv.is_contiguous() and qkv.shape[1] == (num_q_heads + 2 * nkv) * h
    if q_out is None:
        q_out = torch.empty((b, num_q_heads, h), dtype=qkv.dtype, device=qkv.device)
    rc = _lib().axb_rope_append_paged(qkv.data_ptr(), q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                      page_table.data_ptr(), lengths.data_ptr(), b, num_q_heads, nkv, h, page_size,
                                      page_table.shape[1], theta, 1 if apply_rope else 0,
                                      cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_rope_append_paged")  # pylint: disable=protected-access
    return q_out


def swiglu_packed(gu: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, two_f = gu.shape
    f = two_f // 2
    assert gu.is_contiguous()
    if out is None:
        out = torch.empty((rows, f), dtype=gu.dtype, device=gu.device)
    rc = _lib().axb_swiglu_packed(gu.data_ptr(), out.data_ptr(), rows, f, cuda_ops._stream())  # pylint: disable=protected-access
    cuda_ops._check(rc, "axb_swiglu_packed")  # pylint: disable=protected-access
    return out


class OneShotAllReduce:
    """All-reduce of small bf16 vectors over peer memory: every rank stores its partial into
    slot ``rank`` of every peer's staging buffer and raises a flag; every rank then sums its
    slots (optionally on top of a residual).  One instance serves ``sites`` call sites per
    step, each with its own staging and flags, so that no buffer is reused within a step; the
    epoch in ``self.epoch`` (device memory) must be bumped once per step (``begin_step``),
    which also works inside a captured CUDA graph."""

    def __init__(self, numel: int, sites: int, *, group=None, device=None, peers: Optional[list] = None,
                 rank: int = 0):
        from axlearn_b200.parallel import symm

        # With one site a rank that has finished step k could push step k+1 into a peer's slot
        # while that peer still reads it in step k's finish kernel; two sites alternate.
        if sites < 2:
            raise ValueError("OneShotAllReduce needs sites >= 2 (staging is reused across steps)")
        self.numel, self.sites = numel, sites
        if peers is not None:
            # Single-process emulation: `peers[r]` is another instance whose buffers stand in
            # for rank r's memory.
            self.world, self.rank = len(peers) if peers else 1, rank
            self.staging = torch.zeros((sites, max(self.world, 1), numel), dtype=torch.bfloat16, device=device)
            self.flags = torch.zeros((sites, max(self.world, 1)), dtype=torch.int32, device=device)
            self._sym = None
        else:
            import torch.distributed as dist

            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            self.staging, self._sym = symm.symmetric_empty_like_sharded(
                (sites, self.world, numel), torch.bfloat16, group, device)
            self.flags, self._flags_sym = symm.symmetric_empty_like_sharded(
                (sites, self.world), torch.int32, group, device)
            self.flags.zero_()
            self._staging_lists = [[p + s * self.world * numel * 2 for p in self._sym.peer_ptrs] for s in range(sites)]
            self._flag_list = list(self._flags_sym.peer_ptrs)
            self._staging_ptrs = [symm.device_pointer_array(l, device) for l in self._staging_lists]
            self._flag_ptrs = symm.device_pointer_array(self._flag_list, device)
            self._flags_sym.barrier()
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)

    def connect(self, peers: list["OneShotAllReduce"]) -> None:
        """Emulation only: wire the pointer tables to the stand-in peers."""
        dev = self.staging.device
        self._staging_lists = [[p.staging[s].data_ptr() for p in peers] for s in range(self.sites)]
        self._flag_list = [p.flags.data_ptr() for p in peers]
        self._staging_ptrs = [torch.tensor(l, dtype=torch.int64, device=dev) for l in self._staging_lists]
        self._flag_ptrs = torch.tensor(self._flag_list, dtype=torch.int64, device=dev)
        self.world = len(peers)

    def begin_step(self) -> None:
        self.epoch.add_(1)

    def push(self, x: torch.Tensor, site: int) -> None:
        assert x.is_contiguous() and x.numel() == self.numel and x.dtype == torch.bfloat16
        rc = _lib().axb_allreduce_push(x.data_ptr(), self._staging_ptrs[site].data_ptr(), self._flag_ptrs.data_ptr(),
                                       self.counter.data_ptr(), self.epoch.data_ptr(), self.world, self.rank, site,
                                       self.numel, cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_allreduce_push")  # pylint: disable=protected-access

    def gemm_push(self, a: torch.Tensor, b: torch.Tensor, site: int) -> None:
        """``a @ b`` (``[M, K] @ [K, N]``, ``M * N == numel``) with the push half of the all-reduce
        fused into the GEMM's epilogue: rows go straight from the accumulator to every peer."""
        from axlearn_b200.ops import fused_comm

        assert a.shape[0] * b.shape[1] == self.numel
        fused_comm.gemm_allreduce_push(a, b, staging_ptrs=self._staging_lists[site], flag_ptrs=self._flag_list,
                                       counter=self.counter, epoch=self.epoch, rank=self.rank, site=site)

    def finish(self, site: int, *, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
        if out is None:
            out = torch.empty(self.numel, dtype=torch.bfloat16, device=self.staging.device)
        rc = _lib().axb_allreduce_finish(
            self.staging[site].data_ptr(), None if residual is None else residual.data_ptr(), out.data_ptr(),
            self.flags.data_ptr(), self.epoch.data_ptr(), self.world, site, self.numel,
            cuda_ops.status_word(self.staging.device).data_ptr(), cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_allreduce_finish")  # pylint: disable=protected-access
        return out

    def all_reduce(self, x: torch.Tensor, site: int, *, residual=None, out=None) -> torch.Tensor:
        self.push(x, site)
        return self.finish(site, residual=residual, out=out)
