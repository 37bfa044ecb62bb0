"""Honeycrisp: grouped-query decoders with QK-norm and mup-simple learning-rate transfer.

Parity target in the reference: axlearn/experiments/text/gpt/honeycrisp.py -- sizes ``test``,
``85M`` (12 layers, width 768, 12 / 6 heads, FFN 3x) and ``3B`` (26 layers, width 3072, 24 / 8
heads, FFN 8064); vocabulary 48K, sequence length 4096, RoPE theta 5e5, per-head RMSNorm on
queries and keys, RMSNorm eps 1e-5, tied embeddings, AdaStar learner whose matrix updates are
scaled by ``768 / width``.
"""

from __future__ import annotations

from typing import Optional, Union

from axlearn_b200.common import causal_lm
from axlearn_b200.common.attention import (
    FusedGroupedQKVLinear,
    GroupedQueryAttention,
    RepeatedTransformerLayer,
    RoFormerQKVLinear,
    ScaleKey,
    ScaleQuery,
    TransformerLayer,
    scaled_hidden_dim,
)
from axlearn_b200.common.config import InstantiableConfig
from axlearn_b200.common.embedding import TransformerTextEmbeddings
from axlearn_b200.common.layers import RMSNorm
from axlearn_b200.experiments.text.gpt.common import (
    MESH_AXIS_NAMES,
    adastar_learner_config,
    get_trainer_config_fn,
    mesh_shape_from_axes,
    mup_simple_adam_update_transformation,
)
from axlearn_b200.experiments.text.gpt.common import model_config as common_model_config

MODEL_SIZES = ("test", "85M", "3B")
VOCAB_SIZE = 48 * 1024
MAX_SEQUENCE_LENGTH = 4096
_BASE_MODEL_HIDDEN_DIM = 768


def get_trainer_kwargs(model_size: str, *, vocab_size: int = VOCAB_SIZE,
                       max_sequence_length: int = MAX_SEQUENCE_LENGTH, flash_attention: bool = False) -> dict:
    if model_size == "test":
        kw = dict(model_kwargs=dict(num_layers=4, hidden_dim=8, num_heads=4, num_kv_heads=2, vocab_size=32,
                                    ffn_dim=scaled_hidden_dim(scale=8 / 3, round_up_to_multiples_of=16)),
                  learner_kwargs=dict(), max_sequence_length=64, train_batch_size=16, max_step=3000,
                  mesh_shape=mesh_shape_from_axes())
    elif model_size == "85M":
        kw = dict(model_kwargs=dict(num_layers=12, hidden_dim=_BASE_MODEL_HIDDEN_DIM, num_heads=12, num_kv_heads=6,
                                    ffn_dim=scaled_hidden_dim(scale=3.0, round_up_to_multiples_of=32)),
                  learner_kwargs=dict(lr_warmup_steps=5000), train_batch_size=2 ** 20 // max_sequence_length,
                  max_step=600_000, save_every_n_steps=1000, mesh_shape=mesh_shape_from_axes(data=-1))
    elif model_size == "3B":
        kw = dict(model_kwargs=dict(num_layers=26, hidden_dim=128 * 24, num_heads=24, num_kv_heads=8, ffn_dim=8064),
                  learner_kwargs=dict(lr_warmup_steps=5000), train_batch_size=2 ** 20 // max_sequence_length,
                  max_step=600_000, save_every_n_steps=1000, mesh_shape=mesh_shape_from_axes(data=-1, fsdp=8))
    else:
        raise NotImplementedError(f"unknown model size {model_size}")
    model_kwargs = kw.pop("model_kwargs")
    model_kwargs.setdefault("vocab_size", vocab_size)
    learner_kwargs = dict(peak_lr=0.01, alpha=0.005, weight_decay=3.16e-4)
    learner_kwargs.update(kw.pop("learner_kwargs"))
    # mup-simple: matrices learn slower in proportion to the width.
    factor = _BASE_MODEL_HIDDEN_DIM / model_kwargs["hidden_dim"]
    learner_kwargs["adam_update_transformation"] = mup_simple_adam_update_transformation(factor)
    kw.setdefault("max_sequence_length", max_sequence_length)
    return dict(model_cfg=model_config(flash_attention=flash_attention, **model_kwargs),
                learner_cfg=adastar_learner_config(max_step=kw["max_step"], **learner_kwargs),
                vocab_size=model_kwargs["vocab_size"], **kw)


def model_config(*, num_layers: int, hidden_dim: int, num_heads: int, num_kv_heads: int, vocab_size: int,
                 dropout_rate: float = 0.0, ffn_dim: Optional[Union[int, InstantiableConfig]] = None,
                 flash_attention: bool = False, stack_cfg: Optional[InstantiableConfig] = None,
                 scan_chunk: Optional[int] = None) -> causal_lm.Model.Config:
    qkv = RoFormerQKVLinear.default_config().set(
        input_linear=FusedGroupedQKVLinear.default_config().set(num_kv_heads=num_kv_heads), rotary_value=False)
    qkv.rope_pos_emb_layer.theta = 5e5
    norm_cfg = RMSNorm.default_config().set(eps=1e-5, forward_dtype=None)
    layer_cfg = TransformerLayer.default_config()
    if flash_attention:
        from axlearn_b200.common.flash_attention.layer import FlashAttention

        layer_cfg.self_attention.attention = FlashAttention.default_config()
    else:
        layer_cfg.self_attention.attention = GroupedQueryAttention.default_config()
    layer_cfg.self_attention.attention.set(
        query_scale=ScaleQuery.default_config().set(norm=norm_cfg.clone()),
        key_scale=ScaleKey.default_config().set(norm=norm_cfg.clone()))
    layer_cfg.feed_forward.add_dead_neuron_summary = True
    if ffn_dim is None:
        ffn_dim = scaled_hidden_dim(scale=8 / 3, round_up_to_multiples_of=256)
    return common_model_config(
        num_layers=num_layers, hidden_dim=hidden_dim, num_heads=num_heads, vocab_size=vocab_size,
        stack_cfg=stack_cfg if stack_cfg is not None else RepeatedTransformerLayer.default_config(),
        activation_fn=("nn.silu", "linear"), ffn_dim=ffn_dim, normalization=norm_cfg, dropout_rate=dropout_rate,
        emb_cfg=TransformerTextEmbeddings.default_config().set(pos_emb=None), attention_qkv_linear=qkv,
        layer_cfg=layer_cfg, scan_chunk=scan_chunk)


def trainer_configs(train_input_source=None, eval_input_sources=None) -> dict:
    """``honeycrisp-<size>[-flash]``; the input arguments are as in ``gala.trainer_configs``."""

    def make(size, flash):
        def fn():
            kwargs = get_trainer_kwargs(size, flash_attention=flash)
            extra = {}
            if train_input_source is not None:
                extra["train_input_source"] = train_input_source(VOCAB_SIZE, kwargs["max_sequence_length"])
            if eval_input_sources is not None:
                extra["evalers"] = eval_input_sources(vocab_size=VOCAB_SIZE,
                                                      max_sequence_length=kwargs["max_sequence_length"])
            return get_trainer_config_fn(mesh_axis_names=MESH_AXIS_NAMES, **kwargs, **extra)()

        return fn

    out = {}
    for size in MODEL_SIZES:
        out[f"honeycrisp-{size}"] = make(size, False)
        out[f"honeycrisp-{size}-flash"] = make(size, True)
    return out
