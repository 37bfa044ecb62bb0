"""Fuji: a Llama-style decoder-only LM family (RMSNorm, RoPE, SwiGLU, no biases).

Parity targets in the reference (axlearn/experiments/text/gpt/fuji.py): versions and their
vocab / sequence length / RoPE theta (:74-174), ``get_trainer_kwargs`` per model size
(:274-1060), ``model_config`` (:1064-1103), ``trainer_configs`` incl. the ``-flash`` and
``-single-host`` variants (:1106-1255).

Sizes: test, 1B, 3B, 7B, 8B, 70B.  7B: 32 layers, d=4096, 32 heads, ffn 11008, tied output
head.  70B: 80 layers, d=8192, 64 heads / 8 KV heads, ffn 28672, untied head.
"""

from __future__ import annotations

import enum
import itertools
from typing import Any, Callable, Optional, Sequence, Union

import torch

from axlearn_b200.common import causal_lm
from axlearn_b200.common.attention import (
    FusedGroupedQKVLinear,
    FusedQKVLinear,
    GroupedQueryAttention,
    MultiheadAttention,
    RepeatedTransformerLayer,
    RoFormerQKVLinear,
    StackedTransformerLayer,
    scaled_hidden_dim,
)
from axlearn_b200.common.base_layer import RematSpec, nothing_saveable
from axlearn_b200.common.config import InstantiableConfig, config_for_function
from axlearn_b200.common.decoder import LmHead
from axlearn_b200.common.embedding import TransformerTextEmbeddings
from axlearn_b200.common.layers import RMSNorm
from axlearn_b200.common.trainer import SpmdTrainer
from axlearn_b200.common.trainer_config_modifier import (
    ChainConfigModifier,
    MeshShapeModifier,
    RematSpecModifier,
)
from axlearn_b200.experiments.text.gpt.common import (
    MESH_AXIS_NAMES,
    adamw_decoupled_learner_config,
    get_trainer_config_fn,
    mesh_shape_from_axes,
)
from axlearn_b200.experiments.text.gpt.common import model_config as common_model_config

MODEL_SIZES = ("test", "1B", "3B", "7B", "8B", "70B", "405B")


class Version(enum.Enum):
    V1 = 1
    V2 = 2
    V3 = 3
    V3_TIKTOKEN = "3-tiktoken"


VOCAB_SIZE = {Version.V1: 32 * 1024, Version.V2: 32 * 1024, Version.V3: 128 * 1024, Version.V3_TIKTOKEN: 128256}
MAX_SEQUENCE_LENGTH = {Version.V1: 2048, Version.V2: 4096, Version.V3: 8192, Version.V3_TIKTOKEN: 8192}
ROPE_THETA = {Version.V1: 1e4, Version.V2: 1e4, Version.V3: 5e5, Version.V3_TIKTOKEN: 5e5}
# Tokens per batch: 4M for v1/v2, 16M for v3 (reference fuji.py:169-174).
TOKENS_PER_BATCH = {Version.V1: 4 * 2**20, Version.V2: 4 * 2**20, Version.V3: 16 * 2**20, Version.V3_TIKTOKEN: 16 * 2**20}


def full_remat_modifier() -> InstantiableConfig:
    """Per-layer full rematerialisation (keep only the layer input)."""
    return RematSpecModifier.default_config().set(
        remat_policies={"model.decoder.transformer.layer": RematSpec(prevent_cse=False, policy=nothing_saveable)})


def get_trainer_kwargs(
    model_size: str, *, vocab_size: int, version: Version, flash_attention: bool = False,
) -> dict[str, Any]:
    """Hyper-parameters of one Fuji size/version."""
    max_seq = MAX_SEQUENCE_LENGTH[version]
    tokens_per_batch = TOKENS_PER_BATCH[version]
    train_batch_size = tokens_per_batch // max_seq
    # Training budget in tokens (binary "T" = 1024^4): 1T for v1 (1.4T for 70B), 2T for v2, 15T for v3.
    tera = 1024 ** 4
    if version == Version.V1:
        total_tokens = int(1.4 * tera) if model_size == "70B" else tera
    elif version == Version.V2:
        total_tokens = 2 * tera
    else:
        total_tokens = 15 * tera
    max_step = total_tokens // tokens_per_batch
    rope_theta = ROPE_THETA[version]
    gqa = version in (Version.V3, Version.V3_TIKTOKEN)
    common = dict(vocab_size=vocab_size, rope_theta=rope_theta, flash_attention=flash_attention)
    if model_size == "test":
        kw = dict(
            model_kwargs=dict(num_layers=4, hidden_dim=8, ffn_dim=scaled_hidden_dim(scale=8 / 3, round_up_to_multiples_of=16),
                              num_heads=4, num_kv_heads=2 if gqa else None, shared_lm_head=True, **common),
            learner_kwargs=dict(peak_lr=6e-4, weight_decay=0.01),
            max_sequence_length=64, train_batch_size=32, max_step=3000,
            mesh_shape=mesh_shape_from_axes(),
        )
    elif model_size == "1B":
        kw = dict(
            model_kwargs=dict(num_layers=16, hidden_dim=2048, num_heads=32, num_kv_heads=8 if gqa else None,
                              ffn_dim=8192 if gqa else None, shared_lm_head=True, **common),
            learner_kwargs=dict(peak_lr=3e-4, weight_decay=0.1),
            max_sequence_length=max_seq, train_batch_size=train_batch_size, max_step=max_step,
            mesh_shape=mesh_shape_from_axes(data=-1, fsdp=8),
        )
    elif model_size == "3B":
        kw = dict(
            model_kwargs=dict(num_layers=28, hidden_dim=3072, num_heads=24, num_kv_heads=8 if gqa else None,
                              ffn_dim=8192 if gqa else None, shared_lm_head=True, **common),
            learner_kwargs=dict(peak_lr=3e-4, weight_decay=0.1),
            max_sequence_length=max_seq, train_batch_size=train_batch_size, max_step=max_step,
            mesh_shape=mesh_shape_from_axes(data=-1, fsdp=8),
        )
    elif model_size == "7B":
        kw = dict(
            # The feed-forward width stays 8/3 x 4096 rounded up to 256 = 11008 in every version
            # (only the "8B" size of the tiktoken variant widens it to 3.5 x).
            model_kwargs=dict(num_layers=32, hidden_dim=4096, num_heads=32, num_kv_heads=8 if gqa else None,
                              ffn_dim=None, shared_lm_head=True, **common),
            learner_kwargs=dict(peak_lr=3e-4, weight_decay=0.1),
            max_sequence_length=max_seq, train_batch_size=train_batch_size, max_step=max_step,
            mesh_shape=mesh_shape_from_axes(data=-1, fsdp=8),
            mesh_rules=(
                # 8xB200 / 8xH100 single node: pure FSDP over the NVSwitch domain.
                ("gpu-(p5.48xlarge|p4de.24xlarge|a3-highgpu-8g|a4-highgpu-8g|b200)-(8|16|32|64|128|256|512|1024)",
                 ChainConfigModifier.default_config().set(config_modifiers=[
                     MeshShapeModifier.default_config().set(mesh_shape=mesh_shape_from_axes(data=-1, fsdp=8)),
                 ])),
            ),
        )
    elif model_size == "8B":
        kw = dict(
            model_kwargs=dict(num_layers=32, hidden_dim=4096, num_heads=32, num_kv_heads=8,
                              ffn_dim=scaled_hidden_dim(scale=3.5, round_up_to_multiples_of=256),
                              shared_lm_head=False, **common),
            learner_kwargs=dict(peak_lr=3e-4, weight_decay=0.1),
            max_sequence_length=max_seq, train_batch_size=train_batch_size, max_step=max_step,
            mesh_shape=mesh_shape_from_axes(data=-1, fsdp=8),
        )
    elif model_size == "70B":
        kw = dict(
            model_kwargs=dict(num_layers=80, hidden_dim=8192, num_heads=64,
                              num_kv_heads=None if version == Version.V1 else 8,
                              ffn_dim=scaled_hidden_dim(scale=3.5, round_up_to_multiples_of=256),
                              shared_lm_head=False, **common),
            learner_kwargs=dict(peak_lr=1.5e-4, weight_decay=0.1),
            max_sequence_length=max_seq, train_batch_size=train_batch_size, max_step=max_step,
            mesh_shape=mesh_shape_from_axes(fsdp=-1),
            mesh_rules=(
                ("gpu-(a4-highgpu-8g|b200)-8",
                 MeshShapeModifier.default_config().set(mesh_shape=mesh_shape_from_axes(fsdp=4, model=2))),
            ),
        )
    elif model_size == "405B":
        kw = dict(
            model_kwargs=dict(num_layers=126, hidden_dim=16384, num_heads=128, num_kv_heads=8, ffn_dim=53248,
                              shared_lm_head=False, **common),
            learner_kwargs=dict(peak_lr=1.5e-4, weight_decay=0.1),
            max_sequence_length=max_seq, train_batch_size=train_batch_size, max_step=max_step,
            mesh_shape=mesh_shape_from_axes(fsdp=-1),
        )
    else:
        raise NotImplementedError(f"Unknown model size {model_size}")
    mk = kw["model_kwargs"]
    if mk.get("ffn_dim") is None:
        mk["ffn_dim"] = scaled_hidden_dim(scale=8 / 3, round_up_to_multiples_of=256)
    mk.setdefault("vocab_size", vocab_size)
    return kw


def model_config(
    *,
    num_layers: int,
    hidden_dim: int,
    num_heads: int,
    num_kv_heads: Optional[int],
    vocab_size: int,
    rope_theta: float,
    shared_lm_head: bool,
    dropout_rate: float = 0.0,
    ffn_dim: Optional[Union[int, InstantiableConfig]] = None,
    flash_attention: bool = False,
    stack_cfg: Optional[InstantiableConfig] = None,
    scan_chunk: Optional[int] = None,
) -> causal_lm.Model.Config:
    """Fuji model config: pre-norm RMSNorm(eps 1e-5, stats in the activation dtype), RoPE on
    q/k, SwiGLU FFN, fused QKV projection, causal attention."""
    activation_fn = ("nn.silu", "linear")
    if ffn_dim is None:
        ffn_dim = scaled_hidden_dim(scale=8 / 3, round_up_to_multiples_of=256)
    if num_kv_heads:
        atten_cfg = GroupedQueryAttention.default_config()
        atten_input_linear = FusedGroupedQKVLinear.default_config().set(num_kv_heads=num_kv_heads)
    else:
        atten_cfg = MultiheadAttention.default_config()
        atten_input_linear = FusedQKVLinear.default_config()
    if flash_attention:
        from axlearn_b200.common.flash_attention.layer import FlashAttention

        atten_cfg = FlashAttention.default_config()
    atten_qkv_linear = RoFormerQKVLinear.default_config().set(input_linear=atten_input_linear, rotary_value=False)
    atten_qkv_linear.rope_pos_emb_layer.theta = rope_theta
    cfg = common_model_config(
        num_layers=num_layers, hidden_dim=hidden_dim, num_heads=num_heads, vocab_size=vocab_size,
        stack_cfg=stack_cfg if stack_cfg is not None else RepeatedTransformerLayer.default_config(),
        activation_fn=activation_fn, ffn_dim=ffn_dim,
        normalization=RMSNorm.default_config().set(eps=1e-5, forward_dtype=None),
        dropout_rate=dropout_rate, emb_cfg=TransformerTextEmbeddings.default_config().set(pos_emb=None),
        lm_head_cfg=LmHead.default_config() if not shared_lm_head else None,
        attention_cfg=atten_cfg, attention_qkv_linear=atten_qkv_linear, scan_chunk=scan_chunk,
    )
    return cfg


# Which sizes exist in which version (the reference trains no 1B / 3B / 405B on the v1 / v2 recipes
# and names the 4096-wide tiktoken model 8B).
SIZES_BY_VERSION = {
    Version.V1: ("test", "7B", "70B"),
    Version.V2: ("test", "7B", "70B"),
    Version.V3: ("test", "1B", "3B", "7B", "70B", "405B"),
    Version.V3_TIKTOKEN: ("test", "1B", "3B", "8B", "70B", "405B"),
}


def trainer_configs(
    train_input_source: Optional[Callable[..., InstantiableConfig]] = None,
    eval_input_sources: Optional[Callable[..., dict]] = None,
) -> dict[str, Callable[[], SpmdTrainer.Config]]:
    """All named Fuji trainer configs: ``fuji-{size}-v{version}[-flash][-fp8][-single-host]`` plus
    ``fuji-golden-run-test-v{version}`` (the test size for a handful of steps, used to pin
    numerics)."""
    del eval_input_sources
    config_map: dict[str, Callable[[], SpmdTrainer.Config]] = {}
    for version in Version:
        vocab_size = VOCAB_SIZE[version]
        for model_size, flash in itertools.product(SIZES_BY_VERSION[version], (False, True)):
            name = f"fuji-{model_size}-v{version.value}" + ("-flash" if flash else "")
            config_map[name] = _make(model_size, version, vocab_size, flash, train_input_source)
            if model_size != "test":
                config_map[name + "-fp8"] = _make(model_size, version, vocab_size, flash, train_input_source, fp8=True)
            if model_size in ("1B", "3B", "7B", "8B"):
                config_map[name + "-single-host"] = _make(
                    model_size, version, vocab_size, flash, train_input_source, single_host=True)
                config_map[name + "-fp8-single-host"] = _make(
                    model_size, version, vocab_size, flash, train_input_source, single_host=True, fp8=True)
        config_map[f"fuji-golden-run-test-v{version.value}"] = _make(
            "test", version, vocab_size, False, train_input_source, golden_run=True)
    return config_map


def _make(model_size, version, vocab_size, flash, train_input_source, single_host: bool = False, fp8: bool = False,
          golden_run: bool = False):
    def fn() -> SpmdTrainer.Config:
        kw = get_trainer_kwargs(model_size, vocab_size=vocab_size, version=version, flash_attention=flash)
        mk = dict(kw["model_kwargs"])
        max_seq = kw["max_sequence_length"]
        batch = kw["train_batch_size"]
        if single_host:
            # One 8-GPU node: 1/32 of the global batch (32 sequences of 4096 for v2).
            batch = max(8, batch // 32)
        src = None
        if train_input_source is not None:
            src = train_input_source(vocab_size=vocab_size, max_sequence_length=max_seq)
        cfg = get_trainer_config_fn(
            model_cfg=model_config(scan_chunk=8192 if model_size != "test" else None, **mk),
            learner_cfg=adamw_decoupled_learner_config(max_step=kw["max_step"], **kw["learner_kwargs"]),
            max_step=kw["max_step"], train_batch_size=batch, max_sequence_length=max_seq,
            vocab_size=vocab_size, train_input_source=src, mesh_shape=kw["mesh_shape"],
            mesh_axis_names=MESH_AXIS_NAMES, mesh_rules=kw.get("mesh_rules"),
        )()
        if fp8:
            from axlearn_b200.common.trainer_config_modifier import FP8ConfigModifier

            cfg = FP8ConfigModifier.default_config().set(fp8_amax_history_length=128).instantiate()(cfg)
        if golden_run:
            cfg.max_step = 5
        return cfg

    return fn
