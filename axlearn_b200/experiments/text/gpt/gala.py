"""Gala: multi-head decoders with QK-norm and mup-simple, the baseline family for attention
variants.

Parity target in the reference: axlearn/experiments/text/gpt/gala.py -- sizes ``test``, ``85M``,
``302M``, ``1B``, ``7B``; vocabulary 32K, sequence length 4096; RoPE or ALiBi positions;
``norm_structure`` prenorm / hybridnorm for both sub-layers; per-head RMSNorm on queries and keys;
decoupled AdamW with matrix updates scaled by ``768 / width``.
"""

from __future__ import annotations

from typing import Optional, Union

from axlearn_b200.common import causal_lm
from axlearn_b200.common.attention import (
    FusedQKVLinear,
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
    adamw_decoupled_learner_config,
    get_trainer_config_fn,
    mesh_shape_from_axes,
    mup_simple_adam_update_transformation,
)
from axlearn_b200.experiments.text.gpt.common import model_config as common_model_config

MODEL_SIZES = ("test", "85M", "302M", "1B", "7B")
VOCAB_SIZE = 32 * 1024
MAX_SEQUENCE_LENGTH = 4096
_BASE_MODEL_HIDDEN_DIM = 768

def _recipe(model_size: str, max_sequence_length: int) -> dict:
    """Model sizes and training recipes (tokens per batch, steps, learner settings, mesh)."""
    learner_kwargs = dict(peak_lr=0.01, weight_decay=1e-4, lr_warmup_steps=5_000)
    if model_size == "test":
        return dict(model_kwargs=dict(num_layers=4, hidden_dim=8, num_heads=4, vocab_size=32,
                                      ffn_dim=scaled_hidden_dim(scale=8 / 3, round_up_to_multiples_of=16)),
                    learner_kwargs=dict(peak_lr=6e-4, weight_decay=0.01), max_sequence_length=64, train_batch_size=16,
                    max_step=3000, mesh_shape=mesh_shape_from_axes())
    if model_size == "85M":
        return dict(model_kwargs=dict(num_layers=12, hidden_dim=_BASE_MODEL_HIDDEN_DIM, num_heads=12),
                    learner_kwargs=learner_kwargs, train_batch_size=2 ** 20 // max_sequence_length,
                    max_step=400_000, mesh_shape=mesh_shape_from_axes(fsdp=-1))
    if model_size == "302M":
        return dict(model_kwargs=dict(num_layers=24, hidden_dim=64 * 16, num_heads=16),
                    learner_kwargs=learner_kwargs, train_batch_size=2 ** 20 // max_sequence_length,
                    max_step=400_000, mesh_shape=mesh_shape_from_axes(fsdp=-1))
    if model_size == "1B":
        return dict(model_kwargs=dict(num_layers=24, hidden_dim=64 * 32, num_heads=32),
                    learner_kwargs=learner_kwargs, train_batch_size=2 ** 20 // max_sequence_length,
                    max_step=300_000, mesh_shape=mesh_shape_from_axes(fsdp=-1))
    if model_size == "7B":
        return dict(model_kwargs=dict(num_layers=32, hidden_dim=128 * 32, num_heads=32),
                    learner_kwargs=learner_kwargs, train_batch_size=4 * 2 ** 20 // max_sequence_length,
                    max_step=250_000, mesh_shape=mesh_shape_from_axes(fsdp=-1),
                    mesh_rules=(("gpu-.*-(256|512|1024)", mesh_shape_from_axes(data=-1, fsdp=8)),))
    raise NotImplementedError(f"unknown model size {model_size}")


def model_config(*, num_layers: int, hidden_dim: int, num_heads: int, vocab_size: int, dropout_rate: float = 0.0,
                 ffn_dim: Optional[Union[int, InstantiableConfig]] = None, flash_attention: bool = False,
                 norm_structure: str = "prenorm", position_encoding: str = "rope",
                 stack_cfg: Optional[InstantiableConfig] = None,
                 scan_chunk: Optional[int] = None) -> causal_lm.Model.Config:
    if norm_structure not in ("prenorm", "hybridnorm"):
        raise ValueError(f"unsupported norm structure {norm_structure!r}")
    if position_encoding == "rope":
        attention_mask = None
        qkv = RoFormerQKVLinear.default_config().set(input_linear=FusedQKVLinear.default_config(), rotary_value=False)
    elif position_encoding == "alibi":
        from axlearn_b200.common.attention_logit_bias import ALiBiAttentionLogitBiasLayer

        attention_mask = ALiBiAttentionLogitBiasLayer.default_config().set(num_heads=num_heads)
        qkv = FusedQKVLinear.default_config()
    else:
        raise ValueError(f"position encoding {position_encoding!r} is not supported")
    norm_cfg = RMSNorm.default_config().set(eps=1e-5, forward_dtype=None)
    layer_cfg = TransformerLayer.default_config()
    if flash_attention:
        from axlearn_b200.common.flash_attention.layer import FlashAttention

        layer_cfg.self_attention.attention = FlashAttention.default_config()
    layer_cfg.self_attention.attention.set(
        query_scale=ScaleQuery.default_config().set(norm=norm_cfg.clone()),
        key_scale=ScaleKey.default_config().set(norm=norm_cfg.clone()))
    if ffn_dim is None:
        ffn_dim = scaled_hidden_dim(scale=8 / 3, round_up_to_multiples_of=256)
    cfg = common_model_config(
        num_layers=num_layers, hidden_dim=hidden_dim, num_heads=num_heads, vocab_size=vocab_size,
        stack_cfg=stack_cfg if stack_cfg is not None else RepeatedTransformerLayer.default_config(),
        activation_fn=("nn.silu", "linear"), ffn_dim=ffn_dim, normalization=norm_cfg, dropout_rate=dropout_rate,
        emb_cfg=TransformerTextEmbeddings.default_config().set(pos_emb=None), attention_qkv_linear=qkv,
        layer_cfg=layer_cfg, ffn_structure=norm_structure, atten_structure=norm_structure, scan_chunk=scan_chunk)
    cfg.decoder.attention_mask = attention_mask
    return cfg


# Variants generated on top of the base (prenorm + RoPE) configs.
MODEL_SIZE_CONFIG_ARGS_ADDITIONAL = {
    "1B": [dict(norm_structure="hybridnorm", position_encoding="alibi", flash_only=True)],
    "7B": [dict(norm_structure="hybridnorm", position_encoding="alibi")],
}


def get_trainer_kwargs(model_size: str, *, vocab_size: int = VOCAB_SIZE,
                       max_sequence_length: int = MAX_SEQUENCE_LENGTH, norm_structure: str = "prenorm",
                       position_encoding: str = "rope", flash_attention: bool = False) -> dict:
    kw = _recipe(model_size, max_sequence_length)
    model_kwargs = kw.pop("model_kwargs")
    model_kwargs.setdefault("vocab_size", vocab_size)
    # mup-simple: matrices of models wider than the base learn slower in proportion.
    factor = min(_BASE_MODEL_HIDDEN_DIM / model_kwargs["hidden_dim"], 1.0)
    kw["model_cfg"] = model_config(norm_structure=norm_structure, position_encoding=position_encoding,
                                   flash_attention=flash_attention, **model_kwargs)
    kw["learner_cfg"] = adamw_decoupled_learner_config(
        max_step=kw["max_step"], adam_update_transformation=mup_simple_adam_update_transformation(factor),
        **kw.pop("learner_kwargs"))
    kw.setdefault("max_sequence_length", max_sequence_length)
    kw["vocab_size"] = model_kwargs["vocab_size"]
    return kw


def config_name_suffix(*, norm_structure: str, position_encoding: str, enable_flash: bool) -> str:
    parts = []
    if norm_structure != "prenorm":
        parts.append(norm_structure)
    if position_encoding != "rope":
        parts.append(position_encoding)
    if enable_flash:
        parts.append("flash")
    return "-".join(parts)


def trainer_configs(train_input_source=None, eval_input_sources=None) -> dict:
    """``gala-<size>[-hybridnorm-alibi][-flash]``.  ``train_input_source(vocab_size,
    max_sequence_length)`` and ``eval_input_sources(vocab_size=, max_sequence_length=)`` supply the
    inputs; synthetic tokens otherwise."""

    def make(size, flash, norm_structure, position_encoding):
        def fn():
            kwargs = get_trainer_kwargs(size, norm_structure=norm_structure, position_encoding=position_encoding,
                                        flash_attention=flash)
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
        for flash in (False, True):
            base = dict(norm_structure="prenorm", position_encoding="rope")
            for args in [base, *MODEL_SIZE_CONFIG_ARGS_ADDITIONAL.get(size, [])]:
                if args.get("flash_only") and not flash:
                    continue
                suffix = config_name_suffix(norm_structure=args["norm_structure"],
                                            position_encoding=args["position_encoding"], enable_flash=flash)
                out["-".join(p for p in ("gala", size, suffix) if p)] = make(
                    size, flash, args["norm_structure"], args["position_encoding"])
    return out
