"""Dense KV cache ``[B, T, Nkv, H]`` with in-place append.

Parity target: ``KVCache`` in the reference (axlearn/common/kv_cache/kv_cache.py:21-124).  The
reference chooses between a one-hot matmul and dynamic-update-slice because its arrays are
immutable; here the cache is a persistent device buffer and an append is an indexed store
(the CUDA path writes the new rows straight from the QKV-projection epilogue buffer).
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common.kv_cache.base_kv_cache import BaseKVCache, KVState

Tensor = torch.Tensor


class KVCache(BaseKVCache):
    def init_states(self, shape, *, dtype, device=None):
        dt = self._cache_dtype(dtype)
        dims = (shape.batch_size, shape.kv_len, shape.num_kv_heads, shape.per_head_dim)
        return {
            "key": torch.zeros(dims, dtype=dt, device=device),
            "value": torch.zeros(dims, dtype=dt, device=device),
        }

    def extend_step(self, cached_states, *, k_proj, v_proj, key_positions, live_step_len=None, page_pool=None):
        key, value = cached_states["key"], cached_states["value"]
        b, steps = k_proj.shape[:2]
        kv_len = key.shape[1]
        if key_positions.shape[0] == 1 and b > 1:
            key_positions = key_positions.expand(b, -1)
        pos = key_positions.long()
        valid = (pos >= 0) & (pos < kv_len)
        if live_step_len is not None:
            valid = valid & (torch.arange(steps, device=pos.device)[None] < live_step_len[:, None])
        if steps == kv_len and bool((pos[:, 0] == 0).all()) and live_step_len is None:
            key = k_proj.to(key.dtype)
            value = v_proj.to(value.dtype)
        else:
            bidx = torch.arange(b, device=pos.device)[:, None].expand(-1, steps)
            safe = pos.clamp(0, kv_len - 1)
            # Invalid rows rewrite the slot with its current content (a no-op store).
            k_new = torch.where(valid[..., None, None], k_proj.to(key.dtype), key[bidx, safe])
            v_new = torch.where(valid[..., None, None], v_proj.to(value.dtype), value[bidx, safe])
            key = key.index_put((bidx, safe), k_new)
            value = value.index_put((bidx, safe), v_new)
        positions = torch.arange(kv_len, device=pos.device)[None]
        return {"key": key, "value": value}, KVState(k_proj=key, v_proj=value, key_positions=positions)
