"""Autoregressive decoder-only language model.

Parity targets in the reference (axlearn/common/causal_lm.py): loss metrics
``CrossEntropyLossMetrics`` / ``AuxLossMetrics`` / ``CompositeLossMetrics`` (:62-356),
``Model`` (:359) with ``forward`` (:407), ``predict`` (:566), ``score``, ``extract_logits``,
``sample_decode`` / ``beam_search_decode`` (:483-514), chunked loss via ``scan_chunk``
(:637-806), and ``TransformerStackConfig`` helpers (:848-940).

Data parallelism: each rank sees its slice of the global batch.  The loss is normalised by
the *global* number of live targets (a scalar all-reduce over the batch axes), so summing
parameter gradients over those axes — which the FSDP reduce-scatter does — yields exactly the
gradient of the global mean.
"""

from __future__ import annotations

import math
import re
from typing import Any, Optional, Sequence, Union

import torch

from axlearn_b200 import ops
from axlearn_b200.common.attention import (
    BaseStackedTransformerLayer,
    CausalAttentionBias,
    RepeatedTransformerLayer,
    StackedTransformerLayer,
    TransformerLayer,
)
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import (
    REQUIRED,
    InstantiableConfig,
    Required,
    config_class,
)
from axlearn_b200.common.decoder import Decoder
from axlearn_b200.common.loss import cross_entropy
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.module import child_context, nowrap
from axlearn_b200.common.utils import flatten_items
from axlearn_b200.parallel import collectives as coll

Tensor = torch.Tensor

# Mesh axes over which the batch dimension is split.
# Axes over which tokens are split: the batch axes, plus "seq" when sequences are sharded
# (Ulysses-style sequence parallelism).
BATCH_AXES = ("data", "expert", "fsdp", "seq")


def _live_targets(input_batch: dict, target_labels: Tensor) -> Tensor:
    live = input_batch.get("live_targets")
    if live is None:
        live = target_labels >= 0
    return live


class BaseLossMetrics(BaseLayer):
    """Computes ``(loss WeightedSummary, metrics dict)`` from predictions."""

    @config_class
    class Config(BaseLayer.Config):
        pass

    def forward(self, input_batch: dict, *, predict_outputs: dict, module_outputs: dict):
        raise NotImplementedError(type(self))


class CrossEntropyLossMetrics(BaseLossMetrics):
    @config_class
    class Config(BaseLossMetrics.Config):
        z_loss_scale: float = 0.0

    def forward(self, input_batch: dict, *, predict_outputs: dict, module_outputs: dict):
        cfg = self._config
        target_labels = input_batch["target_labels"]
        live = _live_targets(input_batch, target_labels)
        num_local = live.sum().float()
        num_global = coll.all_reduce_scalar(num_local, BATCH_AXES)
        denom = num_global.clamp_min(1.0)
        if "logits" in predict_outputs:
            loss, aux = cross_entropy(
                predict_outputs["logits"], target_labels, live_targets=live,
                z_loss_scale=cfg.z_loss_scale, denominator=denom)
        else:
            loss, aux = ops.lm_head_cross_entropy(
                predict_outputs["hidden_states"], predict_outputs["output_weight"], target_labels,
                live_targets=live, z_loss_scale=cfg.z_loss_scale, denominator=denom,
                chunk_tokens=predict_outputs.get("chunk_tokens", 8192))
        # ``loss`` is this rank's share of the global mean; the reported value is the sum of
        # the shares.
        report = lambda x: coll.all_reduce_scalar(x.detach().float(), BATCH_AXES)
        ce = report(aux["cross_entropy_loss"])
        total = report(loss)
        summaries = {
            "loss": WeightedSummary(total, num_global),
            "cross_entropy_loss": WeightedSummary(ce, num_global),
            "perplexity": WeightedSummary(torch.exp(ce), num_global),
            "accuracy": WeightedSummary(report(aux["accuracy"]), num_global),
            "z_loss": WeightedSummary(report(aux["z_loss"]), num_global),
            "train_live_targets": WeightedSummary(num_global, 1),
        }
        if "target_num_bytes" in input_batch and "per_token_loss" in aux:
            nbytes = coll.all_reduce_scalar(input_batch["target_num_bytes"].sum().float(), BATCH_AXES)
            total_nats = report(aux["per_token_loss"].sum())
            summaries["bits_per_byte"] = WeightedSummary(
                total_nats / nbytes.clamp_min(1.0) / math.log(2), nbytes)
        for k, v in summaries.items():
            self.add_summary(k, v)
        metrics = {"cross_entropy": aux["cross_entropy_loss"], "num_targets": num_global, **aux}
        return WeightedSummary(loss, num_global), metrics


class AuxLossMetrics(BaseLossMetrics):
    """Sums module outputs whose path matches ``aux_loss_regex`` (e.g. MoE balance loss)."""

    @config_class
    class Config(BaseLossMetrics.Config):
        aux_loss_regex: Optional[str] = None

    def forward(self, input_batch: dict, *, predict_outputs: dict, module_outputs: dict):
        cfg = self._config
        if cfg.aux_loss_regex is None:
            return None, {}
        pat = re.compile(cfg.aux_loss_regex)
        hits = [v for k, v in flatten_items(module_outputs) if pat.fullmatch(k) and isinstance(v, Tensor)]
        if not hits:
            zero = torch.zeros((), device=input_batch["target_labels"].device)
            return WeightedSummary(zero, 1), {"aux_loss": zero}
        aux = sum(h.float().mean() for h in hits)
        # Like the cross entropy, the returned loss is this rank's share of the global mean
        # (ranks are weighted by their live targets), so that summing shares over the batch
        # axes gives the mean auxiliary loss and gradients can simply be summed.
        num = _live_targets(input_batch, input_batch["target_labels"]).sum().float()
        num_global = coll.all_reduce_scalar(num, BATCH_AXES)
        share = aux * (num / num_global.clamp_min(1.0))
        total = coll.all_reduce_scalar(share.detach(), BATCH_AXES)
        self.add_summary("aux_loss", WeightedSummary(total, num_global))
        return WeightedSummary(share, num_global), {"aux_loss": total}


class CompositeLossMetrics(BaseLossMetrics):
    """Weighted sum of child metrics' losses."""

    @config_class
    class Config(BaseLossMetrics.Config):
        metrics: dict[str, InstantiableConfig] = {}
        loss_weights: Optional[dict[str, float]] = None
        flatten_metrics: bool = True

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._kids = {name: self._add_child(name, c) for name, c in cfg.metrics.items()}

    def forward(self, input_batch: dict, *, predict_outputs: dict, module_outputs: dict):
        cfg = self._config
        total = None
        weight = None
        all_metrics: dict[str, Any] = {}
        for name, kid in self._kids.items():
            loss, metrics = kid(input_batch, predict_outputs=predict_outputs, module_outputs=module_outputs)
            if cfg.flatten_metrics:
                all_metrics.update(metrics)
            else:
                all_metrics[name] = metrics
            if loss is None:
                continue
            w = 1.0 if cfg.loss_weights is None else cfg.loss_weights.get(name, 1.0)
            total = loss.mean * w if total is None else total + loss.mean * w
            weight = loss.weight if weight is None else weight
        return WeightedSummary(total, weight), all_metrics


def metrics_config(*, z_loss_scale: float = 0.0, aux_loss_regex: Optional[str] = None):
    """Standard LM metrics: cross entropy (+z-loss) plus regex-selected auxiliary losses."""
    return CompositeLossMetrics.default_config().set(
        metrics={
            "lm": CrossEntropyLossMetrics.default_config().set(z_loss_scale=z_loss_scale),
            "aux": AuxLossMetrics.default_config().set(aux_loss_regex=aux_loss_regex),
        }
    )


class Model(BaseModel):
    """Decoder-only LM: ``forward(input_batch) -> (loss, aux)``."""

    @config_class
    class Config(BaseModel.Config):
        decoder: Decoder.Config = Decoder.default_config()
        metrics: InstantiableConfig = metrics_config()
        # Tokens per chunk for the fused head + loss path; None computes full logits.
        scan_chunk: Optional[int] = None
        batch_axis_names: Optional[Sequence[str]] = ("data", "expert", "fsdp")
        seq_axis_names: Optional[Sequence[str]] = "seq"
        # Deprecated aliases kept for config compatibility.
        z_loss_scale: Optional[float] = None
        aux_loss_regex: Optional[str] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("decoder", cfg.decoder)
        metrics = cfg.metrics
        if cfg.z_loss_scale is not None or cfg.aux_loss_regex is not None:
            metrics = metrics_config(z_loss_scale=cfg.z_loss_scale or 0.0, aux_loss_regex=cfg.aux_loss_regex)
        self._add_child("metrics", metrics)

    def forward(self, input_batch: dict, return_aux: bool = False) -> tuple[Tensor, dict]:
        """input_batch: ``input_ids [B, T]``, ``target_labels [B, T]`` (+ optional
        ``input_segment_ids``, ``input_positions``, ``target_num_bytes``, ``live_targets``)."""
        predictions = self.predict(input_batch)
        loss, aux = self._metrics(input_batch, predict_outputs=predictions)
        return loss, (aux if return_aux else {})

    def predict(self, input_batch: dict) -> dict:
        decoder_batch = {**input_batch}
        decoder_batch["positions"] = input_batch.get("input_positions")
        return self.decoder(input_batch=decoder_batch)

    def compute_logits(self, predict_outputs: dict) -> Tensor:
        return self.decoder.compute_logits(predict_outputs)

    def _metrics(self, input_batch: dict, *, predict_outputs: dict) -> tuple[Tensor, dict]:
        cfg = self._config
        target_labels = input_batch["target_labels"]
        pad = cfg.decoder.pad_token_id
        target_labels = torch.where(target_labels == pad, torch.full_like(target_labels, -1), target_labels)
        ctx = self.get_invocation_context()
        outputs = dict(predict_outputs)
        fused = cfg.scan_chunk is not None and "logits" not in outputs
        if fused:
            weight, soft_cap = self.decoder.output_weight()
            if soft_cap is None and self.decoder._logits_modifier is None:  # pylint: disable=protected-access
                outputs["output_weight"] = weight.to(outputs["hidden_states"].dtype)
                outputs["chunk_tokens"] = cfg.scan_chunk
            else:
                fused = False
        if not fused and "logits" not in outputs:
            outputs["logits"] = self.compute_logits(outputs)
        loss, metrics = self.metrics(
            {**input_batch, "target_labels": target_labels},
            predict_outputs=outputs,
            module_outputs=ctx.get_module_outputs(),
        )
        # Metric summaries are reported at model level (not under "metrics/...").
        summaries = ctx.output_collection.summaries
        nested = summaries.pop("metrics", {})
        for _, sub in nested.items():
            if isinstance(sub, dict):
                summaries.update(sub)
        return loss.value(), metrics

    def score(self, input_batch: dict) -> dict:
        predictions = self.predict(input_batch)
        logits = self.compute_logits(predictions)
        target_labels = input_batch["target_labels"]
        live = _live_targets(input_batch, target_labels)
        _, aux = ops.reference.cross_entropy(logits, target_labels, live_targets=live)
        return {"per_token_loss": aux["per_token_loss"], "live_targets": live}

    def extract_logits(self, input_batch: dict) -> Tensor:
        return self.compute_logits(self.predict(input_batch))

    def sample_decode(self, input_batch: dict, **kwargs):
        return self.decoder.sample_decode(input_batch=_decode_batch(input_batch), **kwargs)

    def beam_search_decode(self, input_batch: dict, **kwargs):
        return self.decoder.beam_search_decode(input_batch=_decode_batch(input_batch), **kwargs)


def _decode_batch(input_batch: dict) -> dict:
    out = dict(input_batch)
    if "prefix" in out and "input_ids" not in out:
        out["input_ids"] = out["prefix"]
    return out


def residual_initializer_cfg(num_layers: int, scale: float = 0.02):
    """Init scheme scaling residual-branch output projections by ``1/sqrt(2*num_layers)``."""
    from axlearn_b200.common.param_init import DefaultInitializer, WeightInitializer

    return DefaultInitializer.default_config().set(
        init_by_param_name={
            ".*weight$": WeightInitializer.default_config().set(
                fan=None, distribution="normal", scale=scale / math.sqrt(2 * num_layers))
        }
    )


def gpt_decoder_config(
    stack_cfg, num_layers: int, hidden_dim: int, num_heads: int, vocab_size: int, max_position_embeddings: int,
    activation_function: str = "nn.relu", layer_norm_epsilon: float = 1e-8, dropout_rate: float = 0.0,
    layer_remat=None,
):
    """A GPT-2-style decoder config (reference: axlearn/common/causal_lm.py:870-940): learned
    absolute positions, pre-norm LayerNorm, separate biased q / k / v projections, a 4x
    feed-forward with ``activation_function``, residual-scaled initialisation of the two output
    projections, tied input / output embeddings."""
    from axlearn_b200.common.attention import TransformerLayer
    from axlearn_b200.common.decoder import Decoder
    from axlearn_b200.common.embedding import LearnedPositionalEmbedding, TransformerTextEmbeddings
    from axlearn_b200.common.layers import LayerNorm

    layer_cfg = TransformerLayer.default_config()
    layer_cfg.feed_forward.activation = activation_function
    layer_cfg.feed_forward.norm = LayerNorm.default_config().set(eps=layer_norm_epsilon)
    layer_cfg.feed_forward.hidden_dim = 4 * hidden_dim
    layer_cfg.self_attention.norm = LayerNorm.default_config().set(eps=layer_norm_epsilon)
    layer_cfg.self_attention.attention.causal = True
    layer_cfg.self_attention.attention.num_heads = num_heads
    layer_cfg.self_attention.attention.output_linear.param_init = residual_initializer_cfg(num_layers=num_layers)
    layer_cfg.feed_forward.linear2.param_init = residual_initializer_cfg(num_layers=num_layers)
    layer_cfg.remat_spec = layer_remat
    transformer_cfg = stack_cfg.clone().set(num_layers=num_layers, layer=layer_cfg)
    return Decoder.default_config().set(
        transformer=transformer_cfg, dim=hidden_dim, vocab_size=vocab_size,
        emb=TransformerTextEmbeddings.default_config().set(
            pos_emb=LearnedPositionalEmbedding.default_config().set(shape=(max_position_embeddings,))),
        output_norm=LayerNorm.default_config().set(eps=layer_norm_epsilon), dropout_rate=dropout_rate)
