"""Decoder-only transformer trunk with output head and incremental decoding.

Parity targets in the reference (axlearn/common/decoder.py): ``DecodingLayer`` (:203),
``Decoder`` (:467) with ``forward`` (:644), ``init_states`` (:694), ``prefill_states``
(:715-766), ``extend_step`` (:768-850), ``compute_logits`` (:608-641), ``sample_decode`` /
``beam_search_decode`` (:286-448, :852-919), and ``LmHead`` (:921-957).
"""

from __future__ import annotations

from typing import Any, Callable, Optional, Sequence, Union

import torch

from axlearn_b200 import ops
from axlearn_b200.common.attention import (
    BaseStackedTransformerLayer,
    ForwardMode,
    StackedTransformerLayer,
)
from axlearn_b200.common.base_layer import BaseLayer, FactorizationSpec, ParameterSpec
from axlearn_b200.common.config import (
    REQUIRED,
    InstantiableConfig,
    Required,
    config_class,
    maybe_instantiate,
)
from axlearn_b200.common.embedding import BaseEmbedding, TransformerTextEmbeddings
from axlearn_b200.common.layers import Dropout, LayerNorm, set_dropout_rate_recursively
from axlearn_b200.common.module import Module, child_context, nowrap
from axlearn_b200.parallel import collectives as coll

Tensor = torch.Tensor


class LmHead(BaseLayer):
    """Untied output head: ``logits = x @ weight^T`` with ``weight [vocab, dim]``."""

    @config_class
    class Config(BaseLayer.Config):
        vocab_size: Required[int] = REQUIRED
        embedding_dim: Required[int] = REQUIRED

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.param_partition_spec = (None, "model")
        return cfg

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {
            "weight": ParameterSpec(
                shape=(cfg.vocab_size, cfg.embedding_dim),
                mesh_axes=cfg.param_partition_spec,
                factorization=FactorizationSpec(axes=("row", "col")),
            )
        }

    def _weight(self) -> Tensor:
        cfg = self._config
        spec = cfg.param_partition_spec
        cshape = coll.compute_shape((cfg.vocab_size, cfg.embedding_dim), spec)
        w = coll.unshard_param(self.parameters["weight"], spec, compute_shape=cshape)
        if coll.has_axis(spec[1] if spec else None, "model"):
            w = coll.all_gather(w, "model", dim=1)
        return w

    def forward(self, x: Tensor) -> Tensor:
        w = self._weight()
        return ops.linear(x, w.to(x.dtype).t())

    def weight_for_loss(self) -> Tensor:
        """``[vocab, dim]`` weight for the fused head+loss op."""
        return self._weight()


class DecodingLayer(BaseLayer):
    """Holds decoding hyper-parameters and runs sample / beam search over a decoder."""

    @config_class
    class Config(BaseLayer.Config):
        pass

    def _decoder(self) -> "Decoder":
        return self.parent

    def sample_decode(self, *, input_batch: dict, num_decodes: int = 1, max_sequence_length: int,
                      logits_modifier: Optional[Any] = None, stop_decoding_condition: Optional[Any] = None,
                      temperature: float = 1.0, **kwargs):
        from axlearn_b200.common import decoding

        dec = self._decoder()
        return decoding.sample_decode_with_decoder(
            dec, input_batch=input_batch, num_decodes=num_decodes,
            max_sequence_length=max_sequence_length, logits_modifier=maybe_instantiate(logits_modifier),
            stop_decoding_condition=stop_decoding_condition, prng_key=self.prng_key if self.get_invocation_context().prng_key is not None else None,
            temperature=temperature, **kwargs)

    def beam_search_decode(self, *, input_batch: dict, num_decodes: int, max_sequence_length: int,
                           brevity_penalty: Optional[Callable] = None, **kwargs):
        from axlearn_b200.common import decoding

        return decoding.beam_search_decode_with_decoder(
            self._decoder(), input_batch=input_batch, num_decodes=num_decodes,
            max_sequence_length=max_sequence_length, brevity_penalty=brevity_penalty, **kwargs)


class Decoder(BaseLayer):
    """emb -> transformer -> output_norm -> output_dropout; logits via ``lm_head`` or the
    tied token embedding."""

    @config_class
    class Config(BaseLayer.Config):
        attention_mask: Optional[InstantiableConfig] = None
        vocab_size: Required[int] = REQUIRED
        dim: Required[int] = REQUIRED
        dropout_rate: float = 0.0
        emb: BaseEmbedding.Config = TransformerTextEmbeddings.default_config()
        transformer: BaseStackedTransformerLayer.Config = StackedTransformerLayer.default_config()
        output_norm: Optional[InstantiableConfig] = LayerNorm.default_config()
        output_dropout: Dropout.Config = Dropout.default_config()
        lm_head: Optional[InstantiableConfig] = None
        pad_token_id: int = 0
        eos_token_id: int = 1
        logits_partition_spec: Sequence[Any] = ("data", None, "model")
        hidden_state_partition_spec: Optional[Sequence[Any]] = None
        logits_forward_dtype: Optional[torch.dtype] = None
        output_logits_modifier: Optional[Any] = None
        decoding: DecodingLayer.Config = DecodingLayer.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.logits_forward_dtype not in (None, torch.float32):
            raise ValueError("logits_forward_dtype must be None or float32")
        cfg = cfg.clone()
        _set_dropout_if_none(cfg, cfg.dropout_rate)
        self._add_child("emb", cfg.emb.clone(dim=cfg.dim, vocab_size=cfg.vocab_size))
        self._add_child("transformer", cfg.transformer.clone(input_dim=cfg.dim))
        if cfg.output_norm is not None:
            self._add_child("output_norm", cfg.output_norm.clone(input_dim=cfg.dim))
        self._add_child("output_dropout", cfg.output_dropout)
        if cfg.lm_head is not None:
            self._add_child("lm_head", cfg.lm_head.clone(vocab_size=cfg.vocab_size, embedding_dim=cfg.dim))
        self._add_child("decoding", cfg.decoding)
        self._logits_modifier = maybe_instantiate(cfg.output_logits_modifier)
        if cfg.attention_mask is not None:
            self._add_child("attention_mask", cfg.attention_mask)
        self._decode_key_len: Optional[int] = None

    # ------------------------------------------------------------------ core
    def _forward_for_mode(self, *, mode: ForwardMode, input_batch: dict, cached_states=None,
                          cross_attention_data=None, cross_attention_logit_biases=None,
                          self_attention_logit_biases=None, page_pool=None, max_len=None, **kwargs):
        input_ids = input_batch["input_ids"]
        positions = input_batch.get("positions")
        segment_ids = input_batch.get("input_segment_ids")
        emb_batch = {**input_batch, "inputs": input_ids}
        x = self.emb(emb_batch)
        if "attention_mask" in self._children and self_attention_logit_biases is None:
            self_attention_logit_biases = self._attention_mask_biases(
                mode=mode, input_ids=input_ids, positions=positions, segment_ids=segment_ids,
                cached_states=cached_states, max_len=max_len)
        tkw = dict(
            self_attention_logit_biases=self_attention_logit_biases,
            cross_attention_data=cross_attention_data,
            cross_attention_logit_biases=cross_attention_logit_biases,
        )
        tkw = {k: v for k, v in tkw.items() if v is not None}
        if mode == ForwardMode.FORWARD:
            states = None
            out = self.transformer(x, target_segment_ids=segment_ids, target_positions=positions, **tkw)
        elif mode == ForwardMode.INIT_STATES:
            states, out = self.transformer.init_states(
                time_step=cached_states["time_step"], data=x, page_pool=page_pool, max_len=max_len, **tkw)
            states = {"transformer_state": states}
        else:
            states, out = self.transformer.extend_step(
                cached_states["transformer_state"], x, page_pool=page_pool, **tkw)
            states = {"transformer_state": states}
        h = out.data
        self._add_tensor_stats("outputs", h)
        if "output_norm" in self._children:
            h = self.output_norm(h)
        h = self.output_dropout(h)
        return states, {"hidden_states": h}

    def _attention_mask_biases(self, *, mode, input_ids, positions, segment_ids, cached_states, max_len):
        """Biases of the configured ``attention_mask`` layer (e.g. ALiBi).  Training and prefill see
        the ``[T, T]`` bias of the given tokens; a decoding step sees its rows of the bias over the
        whole cache, whose length was fixed when the cache was created."""
        from axlearn_b200.common.attention_logit_bias import decode_step_bias

        b, t = input_ids.shape
        if mode == ForwardMode.EXTEND_STEP:
            if self._decode_key_len is None:
                raise ValueError("extend_step with an attention_mask needs init_states / prefill_states first")
            return decode_step_bias(self.attention_mask, query_positions=positions, key_len=self._decode_key_len)
        if mode == ForwardMode.INIT_STATES:
            self._decode_key_len = max_len or t
        if positions is None:
            positions = torch.arange(t, device=input_ids.device)[None].expand(b, -1)
        if segment_ids is None:
            segment_ids = torch.ones_like(positions)
        return self.attention_mask(segment_ids=segment_ids, positions=positions)

    def forward(self, input_batch: dict, *, cross_attention_data=None, cross_attention_logit_biases=None,
                **kwargs) -> dict:
        """Returns ``{"hidden_states": [B, T, dim]}``; call ``compute_logits`` for logits."""
        _, out = self._forward_for_mode(
            mode=ForwardMode.FORWARD, input_batch=input_batch,
            cross_attention_data=cross_attention_data,
            cross_attention_logit_biases=cross_attention_logit_biases, **kwargs)
        return out

    def compute_logits(self, forward_outputs: dict) -> Tensor:
        cfg = self._config
        x = forward_outputs["hidden_states"]
        if cfg.logits_forward_dtype is not None:
            x = x.to(cfg.logits_forward_dtype)
        if "lm_head" in self._children:
            logits = self.lm_head(x)
        else:
            logits = self.emb.attend(x)
        if self._logits_modifier is not None:
            logits = self._logits_modifier(logits)
        return logits

    def output_weight(self) -> tuple[Tensor, Optional[float]]:
        """``([vocab, dim] weight, soft_cap)`` of the output head, for fused head+loss."""
        if "lm_head" in self._children:
            return self.lm_head.weight_for_loss(), None
        emb = self.emb
        with child_context("emb"):
            with child_context("token_emb"):
                w = emb.token_emb._weight()  # pylint: disable=protected-access
                if coll.has_axis((emb.token_emb.config.param_partition_spec or (None, None))[1], "model"):
                    w = coll.all_gather(w, "model", dim=1)
        return w, getattr(emb.config, "soft_cap_logits", None)

    # ------------------------------------------------------------------ decoding
    def init_states(self, *, batch_size: int, max_sequence_length: int, dtype=None, device=None) -> dict:
        """Allocates empty caches for ``batch_size`` sequences of up to
        ``max_sequence_length`` tokens."""
        from axlearn_b200.common.utils import TensorSpec

        cfg = self._config
        dtype = dtype or self.dtype()
        spec = _QuerySpec((batch_size, max_sequence_length, cfg.dim), dtype, device)
        states, _ = self.transformer.init_states(time_step=None, data=spec, max_len=max_sequence_length)
        self._decode_key_len = max_sequence_length
        return {
            "transformer_state": states,
            "time_step": torch.zeros(batch_size, dtype=torch.int32, device=device),
        }

    def prefill_states(self, *, time_step: Tensor, input_batch: dict, cross_attention_data=None,
                       cross_attention_logit_biases=None, page_pool=None, max_sequence_length=None):
        """Runs the prompt (``time_step[b]`` = number of valid tokens of row b) and returns
        ``(states, {"hidden_states"})``."""
        states, out = self._forward_for_mode(
            mode=ForwardMode.INIT_STATES, input_batch=input_batch,
            cached_states={"time_step": time_step}, cross_attention_data=cross_attention_data,
            cross_attention_logit_biases=cross_attention_logit_biases, page_pool=page_pool,
            max_len=max_sequence_length)
        states["time_step"] = time_step
        return states, out

    def extend_step(self, *, cached_states: dict, input_ids: Tensor, cross_attention_data=None,
                    cross_attention_logit_biases=None, page_pool=None):
        """Feeds ``input_ids [B, steps]`` at positions ``time_step``..; returns
        ``(states, {"hidden_states", "logits"})``."""
        time_step = cached_states["time_step"]
        steps = input_ids.shape[1]
        positions = time_step[:, None] + torch.arange(steps, device=input_ids.device)[None]
        states, out = self._forward_for_mode(
            mode=ForwardMode.EXTEND_STEP,
            input_batch={"input_ids": input_ids, "positions": positions},
            cached_states=cached_states, cross_attention_data=cross_attention_data,
            cross_attention_logit_biases=cross_attention_logit_biases, page_pool=page_pool)
        states["time_step"] = time_step + steps
        out["logits"] = self.compute_logits(out)
        return states, out

    def sample_decode(self, *, input_batch: dict, **kwargs):
        return self.decoding.sample_decode(input_batch=input_batch, **kwargs)

    def parameter_tree(self) -> dict:
        """This decoder's parameters (for callers that run in a child's context, such as the decode
        engine built behind ``sample_decode``)."""
        return self.state

    def beam_search_decode(self, *, input_batch: dict, **kwargs):
        return self.decoding.beam_search_decode(input_batch=input_batch, **kwargs)


class _QuerySpec:
    """Shape/dtype/device stand-in for a query tensor when only allocating caches."""

    def __init__(self, shape, dtype, device):
        self.shape, self.dtype, self.device = tuple(shape), dtype, device


def _set_dropout_if_none(cfg, rate: float) -> None:
    from axlearn_b200.common.layers import _visit_configs

    def fn(c):
        if "klass" in c and isinstance(c.klass, type) and issubclass(c.klass, Dropout) and c.rate is None:
            c.rate = rate

    _visit_configs(cfg, fn)
