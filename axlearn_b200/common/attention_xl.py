"""Transformer-XL style self-attention with relative positional embeddings.

Parity targets in the reference (axlearn/common/attention.py): ``rel_pos_to_abs_pos`` (:2492),
``xl_attention_logits`` (:2569), ``MultiheadRelativePositionLinear`` and ``MultiheadAttentionXL``
(:2606-2757): logits ``= (q + u) . k + (q + v) . r[key - query]`` where ``r`` is a per-head
projection (``r_proj``, no bias) of sinusoidal embeddings of the relative distance and ``u`` /
``v`` are learned per-head biases; the ``1 / sqrt(head_dim)`` factor applies to the logits
(``ScalePosition.LOGIT``, XLNet) or to the query (``ScalePosition.QUERY``, with an optional
learned per-dim scale: the Lingvo / conformer variant).  Self-attention without KV cache only.
"""

from __future__ import annotations

import enum
from typing import Optional

import torch

from axlearn_b200.common.attention import FusedQKVLinear, MultiheadAttention, MultiheadInputLinear
from axlearn_b200.common.attention_bias import as_attention_bias
from axlearn_b200.common.base_layer import ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.embedding import SinusoidalPositionalEmbedding
from axlearn_b200.common.param_init import constant_initializer

Tensor = torch.Tensor


class MultiheadRelativePositionLinear(MultiheadInputLinear):
    """``[num_positions, D] -> [num_positions, N, H]`` (same weight layout as the input projection)."""

    def forward(self, x: Tensor) -> Tensor:
        y = torch.einsum("ld,dnh->lnh", x, self.parameters["weight"].to(x.dtype))
        if self._config.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        return y


def rel_pos_to_abs_pos(x: Tensor) -> Tensor:
    """``x [..., T, 2T - 1]`` indexed by (query, key - query + T - 1) -> ``[..., T, T]`` indexed
    by (query, key)."""
    t = x.shape[-2]
    assert x.shape[-1] == 2 * t - 1
    q = torch.arange(t, device=x.device)[:, None]
    k = torch.arange(t, device=x.device)[None, :]
    index = (k - q + t - 1).expand(*x.shape[:-2], t, t)
    return torch.gather(x, -1, index)


def xl_attention_logits(*, q_proj: Tensor, k_proj: Tensor, relative_pos_emb: Tensor, u: Tensor, v: Tensor) -> Tensor:
    """``q_proj, k_proj [B, T, N, H]``, ``relative_pos_emb [2T - 1, N, H]`` with entry
    ``key - query + T - 1``, ``u, v [N, H]`` -> logits ``[B, N, T, T]``."""
    term_ac = torch.einsum("btnh,bsnh->bnts", q_proj + u, k_proj)
    term_bd = torch.einsum("btnh,lnh->bntl", q_proj + v, relative_pos_emb)
    return term_ac + rel_pos_to_abs_pos(term_bd)


class MultiheadAttentionXL(MultiheadAttention):
    class ScalePosition(enum.Enum):
        LOGIT = 0
        QUERY = 1

    @config_class
    class Config(MultiheadAttention.Config):
        pos_emb_dim: Optional[int] = None          # default: query_dim
        relative_pos_emb: InstantiableConfig = SinusoidalPositionalEmbedding.default_config()
        relative_pos_linear: InstantiableConfig = MultiheadRelativePositionLinear.default_config().set(bias=False)
        scale_position: Required["MultiheadAttentionXL.ScalePosition"] = REQUIRED

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.scale_position = MultiheadAttentionXL.ScalePosition.LOGIT
        cfg.input_linear = FusedQKVLinear.default_config()
        cfg.input_linear.layer.bias = False
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        if not cfg.query_dim == cfg.key_dim == cfg.value_dim:
            raise ValueError("MultiheadAttentionXL requires query_dim == key_dim == value_dim")
        pos_dim = cfg.pos_emb_dim or cfg.query_dim
        self._add_child("relative_pos_emb", cfg.relative_pos_emb.clone(dim=pos_dim))
        self._add_child("r_proj", cfg.relative_pos_linear.clone(
            model_dim=pos_dim, num_heads=cfg.num_heads, per_head_dim=self.per_head_dim()))

    def _create_layer_parameter_specs(self):
        cfg = self._config
        params = dict(super()._create_layer_parameter_specs())
        for name in ("u_bias", "v_bias"):
            params[name] = ParameterSpec(shape=(cfg.num_heads, self.per_head_dim()), mesh_axes=("model", None),
                                         initializer=constant_initializer(0.0))
        return params

    def forward(self, query: Tensor, *, key=None, value=None, attention_logit_biases=None, segment_ids=None,
                query_positions=None, return_aux=None, **unused):
        if key is not None or value is not None:
            raise ValueError("Both key and value must be None for MultiheadAttentionXL")
        cfg = self._config
        q_proj, k_proj, v_proj = self.i_proj(query)
        q_proj = self.scale_query.apply_per_dim_scale(self.scale_query.apply_norm(q_proj))
        if cfg.scale_position == MultiheadAttentionXL.ScalePosition.QUERY:
            q_proj = self.scale_query.apply_scale_factor(q_proj)
        if "scale_key" in self._children:
            k_proj = self.scale_key(k_proj)
        t = q_proj.shape[1]
        distances = torch.arange(t - 1, -t, -1, device=query.device)           # query - key, descending
        r = self.r_proj(self.relative_pos_emb(distances).to(q_proj.dtype))
        logits = xl_attention_logits(
            q_proj=q_proj.float(), k_proj=k_proj.float(), relative_pos_emb=r.float(),
            u=self.parameters["u_bias"].float(), v=self.parameters["v_bias"].float())
        if cfg.scale_position == MultiheadAttentionXL.ScalePosition.LOGIT:
            logits = self.scale_query.apply_scale_factor(logits)
        bias = as_attention_bias(attention_logit_biases)
        if bias.has_value():
            logits = logits + bias.value().float()
        mask = self._build_mask_bias(t=t, s=t, q_pos=None, k_pos=None)
        if mask is not None:
            logits = logits + mask.value().float()
        if segment_ids is not None:
            same = segment_ids[:, :, None] == segment_ids[:, None, :]
            logits = logits + torch.where(same[:, None], 0.0, -1e9)
        probs = torch.softmax(logits, dim=-1)
        probs = self.dropout(probs)
        context = torch.einsum("bnts,bsnh->btnh", probs.to(v_proj.dtype), v_proj)
        out = self.o_proj(context)
        want_probs = return_aux is not None and "probs" in return_aux
        return self.Output(data=out, probs=probs if want_probs else None, kv_state=None)

    def init_states(self, *args, **kwargs):
        raise NotImplementedError(type(self))

    def extend_step(self, *args, **kwargs):
        raise NotImplementedError(type(self))
