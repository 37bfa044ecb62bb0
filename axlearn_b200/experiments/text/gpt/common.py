"""Shared builders for decoder-only LM experiments.

Parity targets in the reference (axlearn/experiments/text/gpt/common.py): mesh axis names
(:80), ``mesh_shape_from_axes`` (:158-188), ``update_model_remat_config`` (:191-206),
``model_config`` (:209-379), ``adamw_decoupled_learner_config`` (:415-451),
``evaler_config_dict``, ``get_trainer_config_fn`` (:681-800).
"""

from __future__ import annotations

from typing import Any, Callable, Optional, Sequence, Union

import torch

from axlearn_b200.common import causal_lm, learner, optimizers, schedule
from axlearn_b200.common.attention import (
    BaseQKVLinear,
    MultiheadAttention,
    RepeatedTransformerLayer,
    StackedTransformerLayer,
    TransformerLayer,
    build_remat_spec,
    set_double_shard_weights_config,
)
from axlearn_b200.common.checkpointer import every_n_steps_policy
from axlearn_b200.common.evaler import SpmdEvaler
from axlearn_b200.common.evaler import every_n_steps_policy as eval_every_n_steps_policy
from axlearn_b200.common.config import (
    InstantiableConfig,
    config_for_function,
)
from axlearn_b200.common.decoder import Decoder
from axlearn_b200.common.embedding import TransformerTextEmbeddings
from axlearn_b200.common.input_fake import FakeLmInput
from axlearn_b200.common.layers import set_bias_recursively, set_norm_recursively
from axlearn_b200.common.param_init import PARAM_REGEXP_WEIGHT, DefaultInitializer, WeightInitializer
from axlearn_b200.common.trainer import SpmdTrainer
from axlearn_b200.parallel.mesh import mesh_shape_from_axes  # noqa: F401 (re-export)

MESH_AXIS_NAMES = ("pipeline", "data", "expert", "fsdp", "seq", "model")
BATCH_AXIS_NAMES = ("data", "expert", "fsdp")
FSDP_AXIS_NAMES = ("expert", "fsdp", "seq")


def update_model_remat_config(*, stack_cfg, layer_cfg, offload_dst: Optional[str] = None) -> None:
    """Default remat for LM stacks: keep attention projections/context tags (the eager
    runtime keeps layer inputs only)."""
    del offload_dst
    spec = build_remat_spec(stack_cfg.clone(layer=layer_cfg))
    layer_cfg.remat_spec = spec


def model_config(
    *,
    hidden_dim: int,
    num_heads: int,
    num_layers: int,
    vocab_size: int,
    activation_fn: Union[str, Sequence[str]],
    ffn_dim: Union[int, InstantiableConfig],
    normalization: InstantiableConfig,
    dropout_rate: float = 0.0,
    stack_cfg: Optional[InstantiableConfig] = None,
    emb_cfg: Optional[InstantiableConfig] = None,
    lm_head_cfg: Optional[InstantiableConfig] = None,
    layer_cfg: Optional[InstantiableConfig] = None,
    attention_cfg: Optional[InstantiableConfig] = None,
    attention_qkv_linear: Optional[InstantiableConfig] = None,
    attention_kv_cache: Optional[InstantiableConfig] = None,
    z_loss_scale: float = 0.0,
    ffn_structure: str = "prenorm",
    atten_structure: str = "prenorm",
    atten_logit_cap: Optional[float] = None,
    pad_token_id: Optional[int] = None,
    eos_token_id: Optional[int] = None,
    ffn_layer_types: Optional[Sequence[str]] = None,
    expert_cfg: Optional[InstantiableConfig] = None,
    moe_ffn_dim: Optional[Union[int, InstantiableConfig]] = None,
    scan_chunk: Optional[int] = None,
) -> causal_lm.Model.Config:
    """Builds a causal LM config from hyper-parameters."""
    stack_cfg = (stack_cfg or RepeatedTransformerLayer.default_config()).clone()
    emb_cfg = (emb_cfg or TransformerTextEmbeddings.default_config()).clone()
    layer_cfg = (layer_cfg or TransformerLayer.default_config()).clone()
    if attention_cfg is not None:
        layer_cfg.self_attention.attention = attention_cfg
    if moe_ffn_dim is None:
        moe_ffn_dim = ffn_dim
    attn = layer_cfg.self_attention.attention
    attn.causal = True
    attn.num_heads = num_heads
    if attention_qkv_linear is not None:
        attn.input_linear = attention_qkv_linear
    if attention_kv_cache is not None:
        attn.kv_cache = attention_kv_cache
    layer_cfg.self_attention.structure = atten_structure
    attn.atten_logit_cap = atten_logit_cap
    if issubclass(stack_cfg.klass, (RepeatedTransformerLayer, StackedTransformerLayer)):
        update_model_remat_config(stack_cfg=stack_cfg, layer_cfg=layer_cfg)
    set_double_shard_weights_config(
        layer_cfg, batch_axis_names=BATCH_AXIS_NAMES, fsdp_axis_names=FSDP_AXIS_NAMES,
        tp_axis_names="model", seq_axis_names="seq")

    def config_dense():
        cfg = layer_cfg.clone()
        cfg.feed_forward.activation = tuple(activation_fn) if not isinstance(activation_fn, str) else activation_fn
        cfg.feed_forward.hidden_dim = ffn_dim
        cfg.feed_forward.structure = ffn_structure
        return cfg

    def config_sparse():
        from axlearn_b200.common.mixture_of_experts import TransformerFeedForwardMoE

        cfg = layer_cfg.clone()
        cfg.feed_forward = (expert_cfg or TransformerFeedForwardMoE.default_config()).clone()
        cfg.feed_forward.activation = tuple(activation_fn) if not isinstance(activation_fn, str) else activation_fn
        cfg.feed_forward.hidden_dim = moe_ffn_dim
        cfg.feed_forward.structure = ffn_structure
        return cfg

    makers = {"dense": config_dense, "sparse": config_sparse}
    if ffn_layer_types is None:
        transformer_cfg = stack_cfg.set(num_layers=num_layers, layer=config_dense())
    else:
        layers = [makers[t]() for t in ffn_layer_types]
        if len(layers) == 1:
            transformer_cfg = stack_cfg.set(num_layers=num_layers, layer=layers[0])
        else:
            # A group of heterogeneous layers repeated num_layers / len(group) times. The
            # group's own layers are not rematerialised individually.
            transformer_cfg = stack_cfg.set(
                num_layers=num_layers // len(layers),
                layer=StackedTransformerLayer.default_config().set(num_layers=len(layers), layer=layers),
            )
    decoder_cfg = Decoder.default_config().set(
        transformer=transformer_cfg, dim=hidden_dim, vocab_size=vocab_size, emb=emb_cfg,
        lm_head=lm_head_cfg, dropout_rate=dropout_rate)
    if pad_token_id is not None:
        decoder_cfg.pad_token_id = pad_token_id
    if eos_token_id is not None:
        decoder_cfg.eos_token_id = eos_token_id
    model_param_init = DefaultInitializer.default_config().set(
        init_by_param_name={
            PARAM_REGEXP_WEIGHT: WeightInitializer.default_config().set(fan="fan_in", distribution="normal")
        })
    cfg = causal_lm.Model.default_config().set(
        decoder=decoder_cfg, param_init=model_param_init, batch_axis_names=None, scan_chunk=scan_chunk)
    if z_loss_scale:
        cfg.metrics = causal_lm.metrics_config(z_loss_scale=z_loss_scale)
    cfg.dtype = torch.float32
    cfg.decoder.logits_partition_spec = (BATCH_AXIS_NAMES, "seq", "model")
    set_bias_recursively(cfg, False)
    set_norm_recursively(cfg, normalization)
    return cfg


def adamw_decoupled_learner_config(
    *, peak_lr: float, max_step: int, weight_decay: float, lr_warmup_steps: int = 2000,
    alpha: float = 0.1, b1: float = 0.9, b2: float = 0.95, eps: float = 1e-8,
    adam_update_transformation: Optional[Any] = None,
) -> learner.Learner.Config:
    """clip_by_global_norm(1) -> decoupled AdamW with a cosine schedule and linear warm-up."""
    update_schedule = config_for_function(schedule.cosine_with_linear_warmup).set(
        peak_lr=1.0, max_step=max_step, warmup_steps=lr_warmup_steps, begin_value=0.0, alpha=alpha)
    optimizer_cfg = config_for_function(optimizers.chain).set(
        args=[
            config_for_function(optimizers.clip_by_global_norm).set(max_norm=1),
            config_for_function(optimizers.adamw_decoupled_optimizer).set(
                learning_rate=peak_lr, b1=b1, b2=b2, eps=eps, update_schedule=update_schedule,
                weight_decay=weight_decay, weight_decay_per_param_scale=None,
                adam_update_transformation=adam_update_transformation),
        ])
    return learner.Learner.default_config().set(optimizer=optimizer_cfg)


def mup_simple_adam_update_transformation(scale_factor: float) -> InstantiableConfig:
    """Scales the Adam update of the transformer's matrices by ``scale_factor`` ("mup-simple",
    arXiv:2309.14322 section 3.2.4): with the base width ``w0`` and the model width ``w`` the
    factor is ``w0 / w``, which keeps a learning rate tuned on the small model valid."""
    return config_for_function(optimizers.scale_update_per_param).set(
        per_param_scale=config_for_function(optimizers.per_param_scale_by_path).set(
            scale_by_path=[
                (".*attention/o_proj/weight", scale_factor),
                (".*attention/i_proj/i_proj/qkv_proj/weight", scale_factor),
                (".*feed_forward/linear1_0/weight", scale_factor),
                (".*feed_forward/linear1_1/weight", scale_factor),
                (".*feed_forward/linear2/weight", scale_factor),
                (".*feed_forward/wi_0_weight", scale_factor),
                (".*feed_forward/wi_1_weight", scale_factor),
                (".*feed_forward/wo_weight", scale_factor),
            ],
            description="scale_by_mup_simple", default_scale=1.0))


def adastar_learner_config(
    *, peak_lr: float, max_step: int, lr_warmup_steps: int = 2000, alpha: float = 0.005,
    weight_decay: float = 3.16e-4, b1: float = 0.95, b2: float = 0.95,
    adam_update_transformation: Optional[Any] = None,
) -> learner.Learner.Config:
    """skip_and_clip_by_global_norm(drop 100, clip 1) around AdaStar in its Adafactor-like
    setting: no gradient momentum, debiased second moment with ``eps_square``, raw updates
    clipped per tensor, momentum on the updates without debiasing."""
    update_schedule = config_for_function(schedule.cosine_with_linear_warmup).set(
        peak_lr=1.0, max_step=max_step, warmup_steps=lr_warmup_steps, begin_value=0.0, alpha=alpha)
    optimizer_cfg = config_for_function(optimizers.skip_and_clip_by_global_norm).set(
        inner=config_for_function(optimizers.adastar_optimizer).set(
            learning_rate=peak_lr, gradient_ema_decay=None, gradient_ema_debias=False,
            gradient_square_ema_decay=b2, gradient_square_ema_debias=True, eps=0.0, eps_square=1e-30,
            raw_update_clipping_threshold=1.0, update_ema_decay=b1, update_ema_debias=False,
            weight_decay=weight_decay, update_schedule=update_schedule,
            adam_update_transformation=adam_update_transformation),
        drop_norm=100, max_norm=1)
    return learner.Learner.default_config().set(optimizer=optimizer_cfg)


def adamw_learner_config(*, peak_lr: float, max_step: int, weight_decay: float, lr_warmup_steps: int = 2000,
                         b1: float = 0.9, b2: float = 0.95, eps: float = 1e-8) -> learner.Learner.Config:
    """clip -> AdamW (decay scaled by lr) with constant lr after warm-up-free start."""
    del max_step, lr_warmup_steps
    optimizer_cfg = config_for_function(optimizers.chain).set(
        args=[
            config_for_function(optimizers.clip_by_global_norm).set(max_norm=1),
            config_for_function(optimizers.adamw_optimizer).set(
                learning_rate=peak_lr, b1=b1, b2=b2, eps=eps, weight_decay=weight_decay),
        ])
    return learner.Learner.default_config().set(optimizer=optimizer_cfg)


def fake_lm_input_config(*, global_batch_size: int, max_sequence_length: int, vocab_size: int,
                         seed: int = 0, is_training: bool = True) -> InstantiableConfig:
    return FakeLmInput.default_config().set(
        global_batch_size=global_batch_size, source_length=max_sequence_length,
        vocab_size=vocab_size, seed=seed, is_training=is_training)


def _as_input(source: InstantiableConfig, *, global_batch_size: int, is_training: bool) -> InstantiableConfig:
    """An ``Input`` config is used as it is (with the recipe's batch size); a source config
    ``(shard_index, shard_count) -> Stage`` is wrapped in a ``PipelineInput``."""
    from axlearn_b200.common.input_base import Input
    from axlearn_b200.common.input_pipeline import PipelineInput

    klass = source.klass if "klass" in source.keys() else None
    if isinstance(klass, type) and issubclass(klass, Input):
        cfg = source.clone()
        if "global_batch_size" in cfg.keys():
            cfg.global_batch_size = global_batch_size
        return cfg
    return PipelineInput.default_config().set(source=source.clone(), global_batch_size=global_batch_size,
                                              is_training=is_training)


def get_trainer_config_fn(
    *,
    model_cfg: causal_lm.Model.Config,
    learner_cfg: learner.Learner.Config,
    max_step: int,
    train_batch_size: int,
    max_sequence_length: int,
    vocab_size: int,
    train_input_source: Optional[InstantiableConfig] = None,
    evalers: Optional[dict[str, InstantiableConfig]] = None,
    mesh_shape: Sequence[int],
    mesh_axis_names: Sequence[str] = MESH_AXIS_NAMES,
    mesh_rules: Optional[Sequence[tuple[str, Any]]] = None,
    eval_every_n_steps: int = 5000,
    eval_batch_size: Optional[int] = None,
    keep_every_n_steps: int = 50_000,
    save_every_n_steps: Optional[int] = None,
    train_dtype: Optional[torch.dtype] = torch.bfloat16,
) -> Callable[[], SpmdTrainer.Config]:
    """Returns a function producing the trainer config (configs are code)."""

    def config_fn() -> SpmdTrainer.Config:
        cfg = SpmdTrainer.default_config().set(name="gpt_trainer")
        cfg.model = model_cfg.clone()
        cfg.learner = learner_cfg.clone()
        cfg.max_step = max_step
        cfg.train_dtype = train_dtype
        cfg.input = _as_input(train_input_source, global_batch_size=train_batch_size, is_training=True) \
            if train_input_source is not None else fake_lm_input_config(
                global_batch_size=train_batch_size, max_sequence_length=max_sequence_length, vocab_size=vocab_size)
        cfg.evalers = {}
        for name, ev in (evalers or {}).items():
            klass = ev.klass if isinstance(ev, InstantiableConfig) and "klass" in ev.keys() else None
            if isinstance(klass, type) and issubclass(klass, SpmdEvaler):
                cfg.evalers[name] = ev.clone()
            else:   # an input source: evaluate the model's own metrics on it
                cfg.evalers[name] = SpmdEvaler.default_config().set(
                    input=_as_input(ev, global_batch_size=eval_batch_size or train_batch_size, is_training=False),
                    eval_policy=config_for_function(eval_every_n_steps_policy).set(n=eval_every_n_steps))
        cfg.checkpointer.save_policy = config_for_function(every_n_steps_policy).set(
            n=save_every_n_steps or min(eval_every_n_steps, 5_000))
        cfg.checkpointer.keep_every_n_steps = min(max_step, keep_every_n_steps)
        cfg.checkpointer.keep_last_n = 3
        cfg.summary_writer.write_every_n_steps = min(eval_every_n_steps, 100)
        cfg.summary_writer.max_queue = 1000
        cfg.mesh_shape = tuple(mesh_shape)
        cfg.mesh_axis_names = tuple(mesh_axis_names)
        cfg.mesh_rules = mesh_rules
        cfg.batch_axis_names = BATCH_AXIS_NAMES
        return cfg

    return config_fn
