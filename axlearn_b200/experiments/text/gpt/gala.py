"""Gala: multi-head decoders with QK-norm and mup-simple, the baseline family for attention
variants.

Parity target in the reference: axlearn/experiments/text/gpt/gala.py -- sizes ``test``, ``85M``,
``302M``, ``1B``, ``7B``; vocabulary 32K, sequence length 4096; RoPE (or ALiBi, not built here);
``norm_structure`` prenorm / hybridnorm for both sub-layers; per-head RMSNorm on queries and keys;
AdaStar learner with matrix updates scaled by ``768 / width``.
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
    adastar_learner_config,
    get_trainer_config_fn,
    mesh_shape_from_axes,
    mup_simple_adam_update_transformation,
)
from axlearn_b200.experiments.text.gpt.common import model_config as common_model_config

MODEL_SIZES = ("test", "85M", "302M", "1B", "7B")
VOCAB_SIZE = 32 * 1024
MAX_SEQUENCE_LENGTH = 4096
_BASE_MODEL_HIDDEN_DIM = 768

_SIZES = {
    "test": dict(num_layers=4, hidden_dim=8, num_heads=4, vocab_size=32,
                 ffn_dim=scaled_hidden_dim(scale=8 / 3, round_up_to_multiples_of=16)),
    "85M": dict(num_layers=12, hidden_dim=768, num_heads=12),
    "302M": dict(num_layers=24, hidden_dim=1024, num_heads=16),
    "1B": dict(num_layers=24, hidden_dim=2048, num_heads=16),
    "7B": dict(num_layers=32, hidden_dim=4096, num_heads=32),
}


def model_config(*, num_layers: int, hidden_dim: int, num_heads: int, vocab_size: int, dropout_rate: float = 0.0,
                 ffn_dim: Optional[Union[int, InstantiableConfig]] = None, flash_attention: bool = False,
                 norm_structure: str = "prenorm", position_encoding: str = "rope",
                 stack_cfg: Optional[InstantiableConfig] = None,
                 scan_chunk: Optional[int] = None) -> causal_lm.Model.Config:
    if position_encoding != "rope":
        raise NotImplementedError(f"position encoding {position_encoding!r} (only 'rope' is built)")
    if norm_structure not in ("prenorm", "hybridnorm"):
        raise ValueError(f"unsupported norm structure {norm_structure!r}")
    qkv = RoFormerQKVLinear.default_config().set(input_linear=FusedQKVLinear.default_config(), rotary_value=False)
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
    return common_model_config(
        num_layers=num_layers, hidden_dim=hidden_dim, num_heads=num_heads, vocab_size=vocab_size,
        stack_cfg=stack_cfg if stack_cfg is not None else RepeatedTransformerLayer.default_config(),
        activation_fn=("nn.silu", "linear"), ffn_dim=ffn_dim, normalization=norm_cfg, dropout_rate=dropout_rate,
        emb_cfg=TransformerTextEmbeddings.default_config().set(pos_emb=None), attention_qkv_linear=qkv,
        layer_cfg=layer_cfg, ffn_structure=norm_structure, atten_structure=norm_structure, scan_chunk=scan_chunk)


def get_trainer_kwargs(model_size: str, *, vocab_size: int = VOCAB_SIZE,
                       max_sequence_length: int = MAX_SEQUENCE_LENGTH, norm_structure: str = "prenorm") -> dict:
    model_kwargs = dict(_SIZES[model_size])
    model_kwargs.setdefault("vocab_size", vocab_size)
    small = model_size == "test"
    max_step = 3000 if small else 500_000
    factor = _BASE_MODEL_HIDDEN_DIM / model_kwargs["hidden_dim"]
    learner_cfg = adastar_learner_config(
        peak_lr=0.01, max_step=max_step, lr_warmup_steps=2000 if small else 5000,
        adam_update_transformation=mup_simple_adam_update_transformation(factor))
    return dict(
        model_cfg=model_config(norm_structure=norm_structure, **model_kwargs), learner_cfg=learner_cfg,
        max_step=max_step, train_batch_size=16 if small else 4 * 2 ** 20 // max_sequence_length,
        max_sequence_length=64 if small else max_sequence_length, vocab_size=model_kwargs["vocab_size"],
        mesh_shape=mesh_shape_from_axes() if small else mesh_shape_from_axes(data=-1, fsdp=8))


def trainer_configs() -> dict:
    def make(size, structure):
        def fn():
            return get_trainer_config_fn(mesh_axis_names=MESH_AXIS_NAMES,
                                         **get_trainer_kwargs(size, norm_structure=structure))()

        return fn

    out = {}
    for size in MODEL_SIZES:
        out[f"gala-{size}"] = make(size, "prenorm")
        out[f"gala-{size}-hybridnorm"] = make(size, "hybridnorm")
    return out
