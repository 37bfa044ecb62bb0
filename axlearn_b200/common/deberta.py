"""DeBERTa v2: disentangled self-attention over content and bucketed relative positions.

Reference: axlearn/common/deberta.py (log bucketing :26-72, ``deberta_relative_position_bucket``
:75, ``DisentangledSelfAttention`` :116-288, ``DeBERTaV2RelativePositionalEmbedding`` :291,
``DeBERTaV2Encoder`` :315, config builders :351-520).

Logits are ``(c2c + c2p + p2c) / sqrt(d * (1 + number of position terms))``: content-to-content
plus, per head, the query against projected position embeddings gathered at bucket(i - j), and
the key against projected position embeddings gathered at bucket(j - i).  All layers read one
relative-position table shared by the encoder.
"""

from __future__ import annotations

import enum
import math
from typing import Optional, Sequence

import torch

from axlearn_b200.common.attention import (
    MultiheadAttention,
    MultiheadInputLinear,
    QKVLinear,
    RepeatedTransformerLayer,
    scaled_hidden_dim,
)
from axlearn_b200.common.attention_bias import as_attention_bias
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.encoder import BertModel, Encoder, bert_embedding_config, bert_model_config
from axlearn_b200.common.layers import Dropout, Embedding, LayerNorm, RedirectToSharedModule
from axlearn_b200.common.param_init import PARAM_REGEXP_WEIGHT, DefaultInitializer, WeightInitializer

Tensor = torch.Tensor


def _make_log_bucket_position(relative_position: Tensor, *, num_directional_buckets: int, max_distance: int) -> Tensor:
    """Distances up to ``num_directional_buckets // 2`` keep their own bucket; larger ones fall
    into logarithmically growing buckets up to ``max_distance``."""
    if not (max_distance > 1 and num_directional_buckets > 1):
        raise ValueError("max_distance and num_directional_buckets must be at least 2")
    sign = torch.sign(relative_position)
    mid = num_directional_buckets // 2
    abs_pos = torch.maximum(relative_position.abs(), torch.full_like(relative_position, mid - 1))
    log_pos = mid + torch.ceil(
        torch.log(abs_pos.float() / mid) / math.log((max_distance - 1) / mid) * (mid - 1)).to(torch.int64)
    return torch.where(abs_pos <= mid, relative_position, log_pos * sign)


def deberta_relative_position_bucket(*, query_len: int, key_len: int, num_directional_buckets: int,
                                     max_distance: int, device=None) -> Tensor:
    """``[query_len, key_len]`` buckets of ``query - key`` in ``[0, 2 * num_directional_buckets]``."""
    rel = torch.arange(query_len, device=device)[:, None] - torch.arange(key_len, device=device)[None, :]
    return _make_log_bucket_position(rel, num_directional_buckets=num_directional_buckets,
                                     max_distance=max_distance) + num_directional_buckets


class DisentangledAttentionType(enum.Enum):
    C2P = 1      # content (query) to position (key)
    P2C = 2      # position (query) to content (key)


class DisentangledSelfAttention(MultiheadAttention):
    @config_class
    class Config(MultiheadAttention.Config):
        attention_type: Required[Sequence[DisentangledAttentionType]] = REQUIRED
        max_distance: Required[int] = REQUIRED
        num_directional_buckets: Optional[int] = None        # default: max_distance
        pos_emb: Required[InstantiableConfig] = REQUIRED     # provides embeddings()
        pos_emb_dropout: InstantiableConfig = Dropout.default_config()
        pos_q_proj: Optional[InstantiableConfig] = None
        pos_k_proj: Optional[InstantiableConfig] = None

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.input_linear = QKVLinear.default_config()
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        types = list(cfg.attention_type)
        if any(not isinstance(t, DisentangledAttentionType) for t in types):
            raise ValueError(f"invalid attention_type {types}")
        if len(set(types)) != len(types):
            raise ValueError(f"duplicate attention_type {types}")
        self._types = set(types)
        self._add_child("pos_emb", cfg.pos_emb)
        self._add_child("pos_emb_dropout", cfg.pos_emb_dropout)
        if hasattr(self.i_proj, "q_proj"):
            self._share_with_descendants(self.i_proj.q_proj, shared_module_name="q_proj")
            self._share_with_descendants(self.i_proj.k_proj, shared_module_name="k_proj")

        def own(bias):
            return MultiheadInputLinear.default_config().set(
                model_dim=self.hidden_dim(), num_heads=cfg.num_heads, per_head_dim=self.per_head_dim(), bias=bias)

        if DisentangledAttentionType.C2P in self._types:
            self._add_child("pos_k_proj", cfg.pos_k_proj or own(True))
        if DisentangledAttentionType.P2C in self._types:
            self._add_child("pos_q_proj", cfg.pos_q_proj or own(False))

    def num_directional_buckets(self) -> int:
        cfg = self._config
        return cfg.num_directional_buckets or cfg.max_distance

    def _scores(self, q: Tensor, k: Tensor) -> Tensor:
        """``[B, T, N, H] x [B or 1, S, N, H] -> [B, N, T, S]`` with the DeBERTa scale."""
        scale = (1 + len(self._types)) ** -0.5
        q = self.scale_query(q * scale)
        if "scale_key" in self._children:
            k = self.scale_key(k)
        return torch.einsum("btnh,bsnh->bnts", q.float(), k.float().expand(q.shape[0], -1, -1, -1))

    def disentangled_attention_bias(self, *, q_proj: Tensor, k_proj: Tensor,
                                    relative_pos_emb: Optional[Tensor] = None,
                                    relative_pos: Optional[Tensor] = None) -> Tensor:
        """Position terms ``[B, N, T, T]``."""
        if q_proj.shape[1] != k_proj.shape[1]:
            raise NotImplementedError("disentangled attention needs query_len == key_len")
        cfg = self._config
        nb = self.num_directional_buckets()
        if relative_pos_emb is None:
            relative_pos_emb = self.pos_emb_dropout(self.pos_emb.embeddings())
        if relative_pos is None:
            relative_pos = deberta_relative_position_bucket(
                query_len=q_proj.shape[1], key_len=k_proj.shape[1], num_directional_buckets=nb,
                max_distance=cfg.max_distance, device=q_proj.device)[None]
        emb = relative_pos_emb[: 2 * nb][None].to(q_proj.dtype)            # [1, 2nb, D]
        rel = relative_pos[:, None]                                        # [B or 1, 1, T, T]
        score = 0
        if DisentangledAttentionType.C2P in self._types:
            c2p = self._scores(q_proj, self.pos_k_proj(emb))               # [B, N, T, 2nb]
            idx = rel.clamp(0, 2 * nb - 1).expand(c2p.shape[0], c2p.shape[1], -1, -1)
            score = score + torch.gather(c2p, -1, idx)
        if DisentangledAttentionType.P2C in self._types:
            p2c = self._scores(k_proj, self.pos_q_proj(emb))               # [B, N, S, 2nb]
            idx = (2 * nb - rel).clamp(0, 2 * nb - 1).expand(p2c.shape[0], p2c.shape[1], -1, -1)
            score = score + torch.gather(p2c, -1, idx).transpose(-1, -2)
        return score

    def forward(self, query: Tensor, *, key=None, value=None, attention_logit_biases=None, segment_ids=None,
                query_positions=None, return_aux=None, **unused):
        if key is not None or value is not None:
            raise ValueError("DisentangledSelfAttention is self-attention only")
        q_proj, k_proj, v_proj = self.i_proj(query)
        logits = self._scores(q_proj, k_proj) + self.disentangled_attention_bias(q_proj=q_proj, k_proj=k_proj)
        bias = as_attention_bias(attention_logit_biases)
        if bias.has_value():
            logits = logits + bias.value().float()
        t = query.shape[1]
        mask = self._build_mask_bias(t=t, s=t, q_pos=None, k_pos=None)
        if mask is not None:
            logits = logits + mask.value().float()
        if segment_ids is not None:
            same = segment_ids[:, :, None] == segment_ids[:, None, :]
            logits = logits + torch.where(same[:, None], 0.0, -1e9)
        probs = self.dropout(torch.softmax(logits, dim=-1))
        context = torch.einsum("bnts,bsnh->btnh", probs.to(v_proj.dtype), v_proj)
        want_probs = return_aux is not None and "probs" in return_aux
        return self.Output(data=self.o_proj(context), probs=probs if want_probs else None, kv_state=None)

    def init_states(self, *args, **kwargs):
        raise NotImplementedError(type(self))

    def extend_step(self, *args, **kwargs):
        raise NotImplementedError(type(self))


class DeBERTaV2RelativePositionalEmbedding(Embedding):
    """The relative-position table, layer-normalised before use."""

    @config_class
    class Config(Embedding.Config):
        norm: InstantiableConfig = LayerNorm.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("norm", cfg.norm.clone(input_dim=cfg.dim))

    def embeddings(self) -> Tensor:
        return self.norm(super().embeddings())


class DeBERTaV2Encoder(Encoder):
    """A BERT encoder whose attention layers share ``relative_pos_emb``."""

    @config_class
    class Config(Encoder.Config):
        relative_pos_emb: InstantiableConfig = DeBERTaV2RelativePositionalEmbedding.default_config()

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.transformer = RepeatedTransformerLayer.default_config()
        cfg.transformer.layer.self_attention.attention = DisentangledSelfAttention.default_config().set(
            pos_emb=RedirectToSharedModule.default_config().set(
                shared_module="relative_pos_emb", method_map=dict(embeddings="embeddings")))
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("relative_pos_emb", cfg.relative_pos_emb.clone(dim=cfg.dim))
        self._share_with_descendants(self.relative_pos_emb, shared_module_name="relative_pos_emb")


def deberta_v2_self_attention_config(
        *, num_heads: int, max_distance: int, hidden_dropout: float = 0.1, attention_dropout: float = 0.1,
        share_projections: bool = True, num_directional_buckets: Optional[int] = None,
        attention_type: Sequence[DisentangledAttentionType] = (DisentangledAttentionType.P2C,
                                                               DisentangledAttentionType.C2P),
        base_cfg: Optional[InstantiableConfig] = None) -> InstantiableConfig:
    """With ``share_projections`` the position projections are the content q / k projections."""
    cfg = base_cfg.clone() if base_cfg is not None else DisentangledSelfAttention.default_config()
    cfg.set(num_heads=num_heads, max_distance=max_distance, num_directional_buckets=num_directional_buckets,
            attention_type=tuple(attention_type))
    cfg.dropout.rate = attention_dropout
    cfg.pos_emb_dropout.rate = hidden_dropout
    if share_projections:
        if cfg.input_linear.klass is not QKVLinear:
            raise ValueError("shared projections need separate q / k / v projections")
        cfg.pos_q_proj = RedirectToSharedModule.default_config().set(shared_module="q_proj")
        cfg.pos_k_proj = RedirectToSharedModule.default_config().set(shared_module="k_proj")
    return cfg


def deberta_v2_encoder_config(*, dim: int, vocab_size: int, num_layers: int, max_distance: int,
                              max_position_embeddings: Optional[int] = None,
                              num_directional_buckets: Optional[int] = None,
                              base_cfg: Optional[InstantiableConfig] = None,
                              stack_cls: Optional[type] = None) -> InstantiableConfig:
    cfg = base_cfg.clone() if base_cfg is not None else DeBERTaV2Encoder.default_config()
    cfg.set(vocab_size=vocab_size, dim=dim)
    cfg.relative_pos_emb.set(num_embeddings=(num_directional_buckets or max_distance) * 2)
    if stack_cls is not None:
        cfg.transformer = stack_cls.default_config().set(layer=cfg.transformer.layer)
    cfg.transformer.set(num_layers=num_layers)
    cfg.transformer.layer.self_attention.set(structure="postnorm")
    cfg.transformer.layer.feed_forward.set(structure="postnorm", activation="nn.gelu", hidden_dim=scaled_hidden_dim(4))
    cfg.emb = bert_embedding_config(max_position_embeddings=max_position_embeddings, layer_norm_epsilon=1e-7)
    return cfg


def deberta_v2_model_config(*, encoder_cfg: InstantiableConfig,
                            head_cfg: Optional[InstantiableConfig] = None) -> InstantiableConfig:
    cfg = bert_model_config(vocab_size=encoder_cfg.vocab_size, hidden_dim=encoder_cfg.dim, head_cfg=head_cfg)
    cfg.encoder = encoder_cfg
    cfg.param_init = DefaultInitializer.default_config().set(init_by_param_name={
        PARAM_REGEXP_WEIGHT: WeightInitializer.default_config().set(fan=None, scale=0.02, distribution="normal")})
    return cfg
