"""Dual-encoder retrieval models over text embeddings.

Reference: axlearn/common/text_dual_encoder.py (``TextEmbeddingStreamEncoder`` :55,
``flatten_and_concat_embeddings`` :148, ``TextEmbeddingAsymmetricContrastiveLossLayer`` :274,
``RankingPairwiseLossLayer`` :342, ``FLOPsLossLayer`` :412, ``TextEmbeddingDualEncoder`` :509).

Batch layout: ``input_batch[<encoder name>]`` holds ``positive_input_ids`` (and optionally
``negative_input_ids`` / ``pairwise_loss_input_ids``) of shape ``[batch, inputs per example,
length]`` plus the matching ``*_paddings [batch, inputs per example]`` (1 = padded input).  A
tower replaces ids by ``*_embeddings [batch, inputs per example, dim]``.
"""

from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

from axlearn_b200.common import schedule
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.loss import (
    asymmetric_contrastive_loss_from_logits,
    contrastive_logits,
    flops_loss,
    ranking_pairwise_loss,
)
from axlearn_b200.common.module import child_context
from axlearn_b200.common.multi_stream_model import FusionNetwork, MultiStreamModel, StreamEncoder
from axlearn_b200.common.param_init import ConstantInitializer
from axlearn_b200.common.text_encoder import TEXT_EMBEDDINGS, TextEmbeddingEncoder

Tensor = torch.Tensor

POSITIVE_EMBEDDINGS = "positive_embeddings"
NEGATIVE_EMBEDDINGS = "negative_embeddings"
PAIRWISE_LOSS_EMBEDDINGS = "pairwise_loss_embeddings"
POSITIVE_INPUT_IDS = "positive_input_ids"
NEGATIVE_INPUT_IDS = "negative_input_ids"
PAIRWISE_LOSS_INPUT_IDS = "pairwise_loss_input_ids"
POSITIVE_PADDINGS = "positive_paddings"
NEGATIVE_PADDINGS = "negative_paddings"
PAIRWISE_LOSS_PADDINGS = "pairwise_loss_paddings"
RANKS = "ranks"
FLATTENED_LEFT_EMBEDDINGS = "flattened_left_embeddings"
FLATTENED_RIGHT_EMBEDDINGS = "flattened_right_embeddings"
RIGHT_PADDINGS = "right_paddings"
SIMILARITY_MATRIX = "similarity_matrix"
NUM_VALID_RANKING_PAIRS = "num_valid_ranking_pairs"
TEXT_DUAL_ENCODER_SHARED_MODULE_NAME = "shared_text_encoder"
ENCODING_FIELD_MAP = {
    POSITIVE_EMBEDDINGS: POSITIVE_INPUT_IDS,
    NEGATIVE_EMBEDDINGS: NEGATIVE_INPUT_IDS,
    PAIRWISE_LOSS_EMBEDDINGS: PAIRWISE_LOSS_INPUT_IDS,
}


class TextEmbeddingStreamEncoder(StreamEncoder):
    """Text encoder, then an optional projection and an optional normalisation."""

    @config_class
    class Config(StreamEncoder.Config):
        output_dim: Required[int] = REQUIRED
        encoding_field_map: dict[str, str] = ENCODING_FIELD_MAP
        text_encoder: InstantiableConfig = TextEmbeddingEncoder.default_config()
        hidden_dim: Optional[int] = None
        output_proj: Optional[InstantiableConfig] = None
        output_norm: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        hidden = cfg.hidden_dim if cfg.hidden_dim is not None else cfg.output_dim
        self._add_child("text_encoder", cfg.text_encoder.clone(output_dim=hidden))
        if hidden != cfg.output_dim and cfg.output_proj is None:
            raise ValueError("output_proj is required when hidden_dim != output_dim")
        if cfg.output_proj is not None:
            self._add_child("output_proj", cfg.output_proj.clone(input_dim=hidden, output_dim=cfg.output_dim))
        if cfg.output_norm is not None:
            self._add_child("output_norm", cfg.output_norm)

    def _encode(self, input_ids: Tensor) -> Tensor:
        emb = self.text_encoder(input_ids)[TEXT_EMBEDDINGS]
        if "output_proj" in self._children:
            emb = self.output_proj(emb)
        if "output_norm" in self._children:
            emb = self.output_norm(emb)
        return emb

    def forward(self, input_batch: dict) -> dict:
        out = dict(input_batch)
        for emb_field, ids_field in self._config.encoding_field_map.items():
            ids = input_batch.get(ids_field)
            if ids is None or ids.shape[1] == 0:
                continue
            b, n, t = ids.shape
            with child_context(f"encode_{ids_field}", module=self):
                emb = self._encode(ids.reshape(b * n, t))
            out[emb_field] = emb.squeeze(1).reshape(b, n, -1)
        return out


def flatten_and_concat_embeddings(*, left_positive_embeddings: Tensor, right_positive_embeddings: Tensor,
                                  right_positive_paddings: Tensor,
                                  right_negative_embeddings: Optional[Tensor] = None,
                                  right_negative_paddings: Optional[Tensor] = None) -> dict:
    """Queries ``[n, 1, d] -> [n, d]``; keys = all positives followed by all negatives
    ``[n * (p + q), d]`` with their paddings ``[n * (p + q)]``."""
    d = left_positive_embeddings.shape[-1]
    if left_positive_embeddings.shape[1] != 1:
        raise ValueError("the left encoder contributes one embedding per example")
    if right_positive_embeddings.shape[-1] != d:
        raise ValueError("left and right embedding widths differ")
    right = right_positive_embeddings.reshape(-1, d)
    paddings = right_positive_paddings.reshape(-1)
    if right_negative_embeddings is not None:
        if right_negative_embeddings.shape[-1] != d:
            raise ValueError("left and right embedding widths differ")
        right = torch.cat([right, right_negative_embeddings.reshape(-1, d)], dim=0)
        paddings = torch.cat([paddings, right_negative_paddings.reshape(-1)], dim=0)
    return {FLATTENED_LEFT_EMBEDDINGS: left_positive_embeddings.reshape(-1, d),
            FLATTENED_RIGHT_EMBEDDINGS: right, RIGHT_PADDINGS: paddings}


def _at(batch: dict, path: Union[str, Sequence[str]]) -> dict:
    for k in ([path] if isinstance(path, str) else path):
        batch = batch[k]
    return batch


def flatten_and_concat_embeddings_from_input_batch(*, input_batch: dict, left_encoder_name, right_encoder_name,
                                                   assert_one_positive_from_right_encoder: bool = True) -> dict:
    left, right = _at(input_batch, left_encoder_name), _at(input_batch, right_encoder_name)
    if assert_one_positive_from_right_encoder and right[POSITIVE_EMBEDDINGS].shape[1] != 1:
        raise ValueError("the right encoder contributes one positive embedding per example")
    return flatten_and_concat_embeddings(
        left_positive_embeddings=left[POSITIVE_EMBEDDINGS],
        right_positive_embeddings=right[POSITIVE_EMBEDDINGS],
        right_positive_paddings=right[POSITIVE_PADDINGS],
        right_negative_embeddings=right.get(NEGATIVE_EMBEDDINGS),
        right_negative_paddings=right.get(NEGATIVE_PADDINGS))


class TextEmbeddingAsymmetricContrastiveLossLayer(FusionNetwork):
    """Softmax cross-entropy of every query over all keys of the batch (in-batch positives and
    negatives); keys are not classified over queries."""

    @config_class
    class Config(FusionNetwork.Config):
        left_encoder_name: Required[Union[str, Sequence[str]]] = REQUIRED
        right_encoder_name: Required[Union[str, Sequence[str]]] = REQUIRED
        contrastive_loss_scale_factor: float = 1.0   # 1 / temperature

    def forward(self, input_batch: dict):
        cfg = self._config
        flat = flatten_and_concat_embeddings_from_input_batch(
            input_batch=input_batch, left_encoder_name=cfg.left_encoder_name,
            right_encoder_name=cfg.right_encoder_name)
        sim = contrastive_logits(flat[FLATTENED_LEFT_EMBEDDINGS], flat[FLATTENED_RIGHT_EMBEDDINGS])
        loss = asymmetric_contrastive_loss_from_logits(
            sim, key_paddings=flat[RIGHT_PADDINGS], temperature=1 / cfg.contrastive_loss_scale_factor)
        return loss, {SIMILARITY_MATRIX: sim}


class RankingPairwiseLossLayer(FusionNetwork):
    """Binary cross-entropy on score differences of every pair of graded candidates."""

    @config_class
    class Config(FusionNetwork.Config):
        left_encoder_name: Required[str] = REQUIRED
        right_encoder_name: Required[str] = REQUIRED
        pairwise_loss_scale_factor: float = 1.0

    def forward(self, input_batch: dict):
        cfg = self._config
        left = input_batch[cfg.left_encoder_name][POSITIVE_EMBEDDINGS]
        if left.shape[1] != 1:
            raise ValueError("the left encoder contributes one embedding per example")
        right = input_batch[cfg.right_encoder_name]
        logits = torch.einsum("bid,bjd->bij", left, right[PAIRWISE_LOSS_EMBEDDINGS]).squeeze(1)
        logits = logits * cfg.pairwise_loss_scale_factor
        ranks = right[RANKS] * (1 - right[PAIRWISE_LOSS_PADDINGS].to(right[RANKS].dtype))
        loss, pairs = ranking_pairwise_loss(logits=logits, ranks=ranks,
                                            loss_scale=torch.ones(left.shape[0], device=left.device))
        return loss, {NUM_VALID_RANKING_PAIRS: pairs}


class FLOPsLossLayer(FusionNetwork):
    """FLOPs regulariser on both towers' sparse embeddings with a scheduled weight; the step
    counter is a parameter advanced through state updates."""

    @config_class
    class Config(FusionNetwork.Config):
        left_encoder_name: Required[Union[str, Sequence[str]]] = REQUIRED
        right_encoder_name: Required[Union[str, Sequence[str]]] = REQUIRED
        flops_weight_schedule: Required[InstantiableConfig] = REQUIRED
        left_encoder_flops_loss_weight: float = 1.0
        right_encoder_flops_loss_weight: float = 1.0
        sparsity_threshold: float = 0.0

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._schedule = schedule.as_schedule_fn(cfg.flops_weight_schedule)

    def _create_layer_parameter_specs(self):
        return {"step": ParameterSpec(shape=(), dtype=torch.int32, mesh_axes=(),
                                      initializer=ConstantInitializer.default_config().set(value=0).instantiate(),
                                      weight_decay_scale=0)}

    def forward(self, input_batch: dict):
        cfg = self._config
        flat = flatten_and_concat_embeddings_from_input_batch(
            input_batch=input_batch, left_encoder_name=cfg.left_encoder_name,
            right_encoder_name=cfg.right_encoder_name, assert_one_positive_from_right_encoder=False)
        left_loss, left_count = flops_loss(embeddings=flat[FLATTENED_LEFT_EMBEDDINGS],
                                           sparsity_threshold=cfg.sparsity_threshold)
        right_loss, right_count = flops_loss(embeddings=flat[FLATTENED_RIGHT_EMBEDDINGS],
                                             paddings=flat[RIGHT_PADDINGS],
                                             sparsity_threshold=cfg.sparsity_threshold)
        self.add_summary(f"{cfg.left_encoder_name}_flops_loss", left_loss)
        self.add_summary(f"{cfg.right_encoder_name}_flops_loss", right_loss)
        self.add_summary(f"{cfg.left_encoder_name}_avg_sparsity_count", left_count)
        self.add_summary(f"{cfg.right_encoder_name}_avg_sparsity_count", right_count)
        step = self.parameters["step"]
        weight = self._schedule(int(step))
        self.add_state_update("step", step + 1)
        return weight * (cfg.left_encoder_flops_loss_weight * left_loss
                         + cfg.right_encoder_flops_loss_weight * right_loss), {}


class TextEmbeddingDualEncoder(MultiStreamModel):
    """Two ``TextEmbeddingStreamEncoder`` towers, each reading ``input_batch[<its name>]``.
    With ``shared_encoder_name`` that tower is shared with descendants so that the other tower
    can be a ``RedirectToSharedModule`` (siamese encoders)."""

    @config_class
    class Config(MultiStreamModel.Config):
        shared_encoder_name: Optional[str] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.shared_encoder_name is not None:
            self._share_with_descendants(self._stream_encoder[cfg.shared_encoder_name],
                                         shared_module_name=TEXT_DUAL_ENCODER_SHARED_MODULE_NAME)

    def _forward_all_stream_encoder(self, input_batch: dict) -> dict:
        for name, enc in self._stream_encoder.items():
            input_batch[name] = enc(input_batch[name])
        return input_batch

    def forward_single_stream_encoder(self, input_batch: dict, encoder_name: str):
        if encoder_name not in self._stream_encoder:
            raise ValueError(f"{encoder_name} is not a stream encoder")
        return self._stream_encoder[encoder_name](input_batch[encoder_name])
