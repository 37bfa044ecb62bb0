"""Paged KV cache: fixed-size pages drawn from a pool, addressed through a page table.

Parity targets in the reference (axlearn/common/kv_cache/paged_kv_cache.py):
``reconstruct_kv`` (:21), ``scatter_update_pages`` (:37), ``PagedKVCache`` (:106-277), and the
scatter kernel (axlearn/common/kv_cache/paged_kv_cache_gpu_kernel.py:16-60).

State: ``key_pages`` / ``value_pages`` of shape ``[num_pages, page_size, Nkv, H]`` (one page
= ``page_size`` consecutive tokens of all KV heads, contiguous, so a page is one TMA box) and
``page_indices [B, pages_per_seq]`` int32; page 0 is reserved as the padding page.  Pages may
come from a ``page_pool`` shared across layers.
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common.config import config_class
from axlearn_b200.common.kv_cache.base_kv_cache import BaseKVCache, KVState

Tensor = torch.Tensor


def reconstruct_kv(page_indices: Tensor, pages: Tensor) -> Tensor:
    """Gathers ``pages[page_indices]`` into ``[B, pages_per_seq * page_size, Nkv, H]``."""
    b, n = page_indices.shape
    g = pages[page_indices.long()]  # [B, n, page, Nkv, H]
    return g.reshape(b, n * pages.shape[1], pages.shape[2], pages.shape[3])


def scatter_update_pages(pages: Tensor, new: Tensor, page_ids: Tensor, offsets: Tensor, valid: Tensor) -> Tensor:
    """Writes ``new[b, s]`` (``[B, steps, Nkv, H]``) to ``pages[page_ids[b,s], offsets[b,s]]``;
    invalid entries are redirected to the padding page 0."""
    pid = torch.where(valid, page_ids, torch.zeros_like(page_ids)).long()
    off = torch.where(valid, offsets, torch.zeros_like(offsets)).long()
    if pages.is_cuda:
        from axlearn_b200.ops import dispatch

        if not dispatch._flags.force_reference:  # pylint: disable=protected-access
            return dispatch._ops().paged_kv_append(pages, new, pid, off)
    return pages.index_put((pid, off), new.to(pages.dtype))


class PagedKVCache(BaseKVCache):
    @config_class
    class Config(BaseKVCache.Config):
        page_size: int = 16
        # Pages allocated per layer when no shared pool is supplied (None = exactly enough).
        num_pages: Optional[int] = None

    def init_states(self, shape, *, dtype, device=None):
        cfg = self._config
        dt = self._cache_dtype(dtype)
        per_seq = -(-shape.kv_len // cfg.page_size)
        total = cfg.num_pages or (1 + shape.batch_size * per_seq)
        dims = (total, cfg.page_size, shape.num_kv_heads, shape.per_head_dim)
        # Default page table: sequence b owns pages 1 + b*per_seq ... (page 0 = padding).
        table = 1 + torch.arange(shape.batch_size * per_seq, device=device, dtype=torch.int32).reshape(
            shape.batch_size, per_seq
        )
        return {
            "key_pages": torch.zeros(dims, dtype=dt, device=device),
            "value_pages": torch.zeros(dims, dtype=dt, device=device),
            "page_indices": table,
        }

    def extend_step(self, cached_states, *, k_proj, v_proj, key_positions, live_step_len=None, page_pool=None):
        cfg = self._config
        kp = cached_states["key_pages"] if page_pool is None else page_pool["key_pages"]
        vp = cached_states["value_pages"] if page_pool is None else page_pool["value_pages"]
        table = cached_states["page_indices"]
        b, steps = k_proj.shape[:2]
        if key_positions.shape[0] == 1 and b > 1:
            key_positions = key_positions.expand(b, -1)
        pos = key_positions.long()
        max_len = table.shape[1] * cfg.page_size
        valid = (pos >= 0) & (pos < max_len)
        if live_step_len is not None:
            valid = valid & (torch.arange(steps, device=pos.device)[None] < live_step_len[:, None])
        safe = pos.clamp(0, max_len - 1)
        page_ids = torch.gather(table.long(), 1, safe // cfg.page_size)
        offsets = safe % cfg.page_size
        kp = scatter_update_pages(kp, k_proj, page_ids, offsets, valid)
        vp = scatter_update_pages(vp, v_proj, page_ids, offsets, valid)
        new_state = dict(cached_states)
        if page_pool is None:
            new_state["key_pages"], new_state["value_pages"] = kp, vp
        else:
            page_pool["key_pages"], page_pool["value_pages"] = kp, vp
        positions = torch.arange(max_len, device=pos.device)[None]
        state = KVState(
            k_proj=None, v_proj=None, key_positions=positions, page_indices=table, pages=(kp, vp)
        )
        return new_state, state


def materialize(kv: KVState) -> KVState:
    """Dense view of a paged KVState (gathers pages); identity for dense states."""
    if kv.k_proj is not None:
        return kv
    kp, vp = kv.pages
    return kv._replace(k_proj=reconstruct_kv(kv.page_indices, kp), v_proj=reconstruct_kv(kv.page_indices, vp))
