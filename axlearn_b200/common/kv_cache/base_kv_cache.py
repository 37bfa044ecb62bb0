"""Interface of KV caches.

Parity targets in the reference: ``KVState`` (axlearn/common/kv_cache/base_kv_cache.py:15)
and ``BaseKVCache`` (:31) with ``init_states`` / ``extend_step``.

Layout differs from the reference on purpose: the reference keeps ``[B, Nkv, H, T]`` (time
last, friendly to TPU lanes); here caches are ``[B, T, Nkv, H]`` so that one token's K/V for
all heads is one contiguous row — appends are a single coalesced store and the decode
kernels stream keys with 16-byte vector loads / TMA boxes of ``[keys, H]``.
"""

from __future__ import annotations

from typing import NamedTuple, Optional

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import config_class

Tensor = torch.Tensor


class KVState(NamedTuple):
    """Projected keys/values with their absolute positions.

    k_proj, v_proj: ``[B, S, Nkv, H]``; key_positions: ``[B|1, S]`` (negative = invalid slot).
    """

    k_proj: Tensor
    v_proj: Tensor
    key_positions: Tensor
    # Paged caches additionally expose the page table so that decode kernels can read pages
    # in place instead of a gathered copy.
    page_indices: Optional[Tensor] = None
    pages: Optional[tuple] = None


class BaseKVCache(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        # Storage dtype of the cache; None = dtype of the projections.
        cache_dtype: Optional[torch.dtype] = None

    class Shape(NamedTuple):
        batch_size: int
        kv_len: int
        num_kv_heads: int
        per_head_dim: int

    def _cache_dtype(self, dtype: torch.dtype) -> torch.dtype:
        return self._config.cache_dtype or dtype

    def init_states(self, shape: "BaseKVCache.Shape", *, dtype: torch.dtype, device=None) -> dict:
        raise NotImplementedError(type(self))

    def extend_step(
        self,
        cached_states: dict,
        *,
        k_proj: Tensor,
        v_proj: Tensor,
        key_positions: Tensor,
        live_step_len: Optional[Tensor] = None,
        page_pool: Optional[dict] = None,
    ) -> tuple[dict, KVState]:
        """Appends ``k_proj``/``v_proj`` (``[B, steps, Nkv, H]``) at ``key_positions``
        (``[B, steps]``) and returns the updated state plus everything attention may read."""
        raise NotImplementedError(type(self))
