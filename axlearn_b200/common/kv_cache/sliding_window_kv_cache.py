"""Ring-buffer KV cache holding only the last ``cached_kv_length`` positions.

Parity target: ``SlidingWindowKVCache`` (axlearn/common/kv_cache/sliding_window_kv_cache.py:
19-177) and ``enable_sliding_window_attention`` (:157).  A token at absolute position ``p``
lives in slot ``p % window``; ``key_positions`` records which absolute position each slot
holds (-1 = empty) so the attention mask can be evaluated on absolute positions.
"""

from __future__ import annotations

import torch

from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.kv_cache.base_kv_cache import BaseKVCache, KVState


class SlidingWindowKVCache(BaseKVCache):
    @config_class
    class Config(BaseKVCache.Config):
        cached_kv_length: Required[int] = REQUIRED

    def init_states(self, shape, *, dtype, device=None):
        dt = self._cache_dtype(dtype)
        w = self._config.cached_kv_length
        dims = (shape.batch_size, w, shape.num_kv_heads, shape.per_head_dim)
        return {
            "key": torch.zeros(dims, dtype=dt, device=device),
            "value": torch.zeros(dims, dtype=dt, device=device),
            "key_positions": torch.full((shape.batch_size, w), -1, dtype=torch.int32, device=device),
        }

    def extend_step(self, cached_states, *, k_proj, v_proj, key_positions, live_step_len=None, page_pool=None):
        key, value, kpos = cached_states["key"], cached_states["value"], cached_states["key_positions"]
        b, steps = k_proj.shape[:2]
        w = key.shape[1]
        if key_positions.shape[0] == 1 and b > 1:
            key_positions = key_positions.expand(b, -1)
        pos = key_positions.long()
        valid = pos >= 0
        if live_step_len is not None:
            valid = valid & (torch.arange(steps, device=pos.device)[None] < live_step_len[:, None])
        # Attention for this step must see both the old window and the new tokens.
        full_k = torch.cat([key, k_proj.to(key.dtype)], dim=1)
        full_v = torch.cat([value, v_proj.to(value.dtype)], dim=1)
        full_pos = torch.cat([kpos.long(), torch.where(valid, pos, -1)], dim=1)
        # Only the last ``w`` new tokens can survive in the ring.
        if steps > w:
            k_proj, v_proj, pos, valid = k_proj[:, -w:], v_proj[:, -w:], pos[:, -w:], valid[:, -w:]
            steps = w
        slot = pos.clamp_min(0) % w
        bidx = torch.arange(b, device=pos.device)[:, None].expand(-1, steps)
        k_new = torch.where(valid[..., None, None], k_proj.to(key.dtype), key[bidx, slot])
        v_new = torch.where(valid[..., None, None], v_proj.to(value.dtype), value[bidx, slot])
        p_new = torch.where(valid, pos.to(kpos.dtype), kpos[bidx, slot])
        new_state = {
            "key": key.index_put((bidx, slot), k_new),
            "value": value.index_put((bidx, slot), v_new),
            "key_positions": kpos.index_put((bidx, slot), p_new),
        }
        return new_state, KVState(k_proj=full_k, v_proj=full_v, key_positions=full_pos)


def enable_sliding_window_attention(cfg, sliding_window_size: int):
    """Configures an attention layer config for causal sliding-window attention with a ring
    cache of matching length."""
    from axlearn_b200.common.attention_bias import SlidingWindowAttentionBias
    from axlearn_b200.common.config import config_for_class

    cfg.kv_cache = SlidingWindowKVCache.default_config().set(cached_kv_length=sliding_window_size)
    cfg.mask = config_for_class(SlidingWindowAttentionBias).set(
        sliding_window_size=sliding_window_size, mask=None, shape=None
    )
    cfg.causal = None
    return cfg
