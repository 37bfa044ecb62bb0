"""Envy: decoder-only LMs with mixture-of-experts feed-forward layers.

Parity target in the reference: axlearn/experiments/text/gpt/envy.py (MoE model family: sparse
and dense layers interleaved by ``ffn_layer_types``, Top2 gating, aux loss collected through
``aux_loss_regex``).  ``MODEL_PRESETS["Mixtral-8x7B"]`` is the Mixtral-style configuration used as
the MoE training benchmark: 32 layers, d_model 4096, 32 query / 8 KV heads, 8 SwiGLU experts of
hidden 14336, top-2 softmax router, capacity factor 2.0, load-balance loss weight 0.01.
"""

from __future__ import annotations

from typing import Optional, Sequence

from axlearn_b200.common import causal_lm
from axlearn_b200.common.attention import (
    FusedGroupedQKVLinear,
    FusedQKVLinear,
    GroupedQueryAttention,
    MultiheadAttention,
    RepeatedTransformerLayer,
    RoFormerQKVLinear,
)
from axlearn_b200.common.config import InstantiableConfig
from axlearn_b200.common.decoder import LmHead
from axlearn_b200.common.embedding import TransformerTextEmbeddings
from axlearn_b200.common.layers import RMSNorm
from axlearn_b200.common.mixture_of_experts import (
    Top2Gating,
    TopKDropFreeGating,
    TopKGating,
    TransformerFeedForwardDropFreeMoE,
    TransformerFeedForwardMoE,
)
from axlearn_b200.experiments.text.gpt.common import model_config as common_model_config

MODEL_PRESETS = {
    "test": dict(num_layers=2, hidden_dim=64, num_heads=4, num_kv_heads=2, num_experts=4, moe_ffn_dim=128,
                 vocab_size=512, num_groups=2),
    # The reference's Switch-Transformer-style sizes: dense and sparse layers alternate, hybrid-norm
    # feed-forward, per-head RMSNorm on queries and keys, 2 routing groups, capacity factor 2.
    "Switch-Base": dict(num_layers=12, hidden_dim=12 * 128, num_heads=12, num_kv_heads=12, num_experts=128,
                        moe_ffn_dim=4 * 12 * 128, vocab_size=32768, num_groups=2, ffn_layer_types=("dense", "sparse"),
                        ffn_structure="hybridnorm", qk_norm=True, shared_lm_head=True, rope_theta=5e5, z_loss_scale=1e-6),
    "Switch-Large": dict(num_layers=24, hidden_dim=16 * 128, num_heads=16, num_kv_heads=16, num_experts=128,
                         moe_ffn_dim=4 * 16 * 128, vocab_size=32768, num_groups=2, ffn_layer_types=("dense", "sparse"),
                         ffn_structure="hybridnorm", qk_norm=True, shared_lm_head=True, rope_theta=5e5, z_loss_scale=1e-6),
    "Switch-XXL": dict(num_layers=24, hidden_dim=64 * 128, num_heads=64, num_kv_heads=8, num_experts=64,
                       moe_ffn_dim=int(2.5 * 64 * 128), vocab_size=32768, num_groups=2,
                       ffn_layer_types=("dense", "sparse"), ffn_structure="hybridnorm", qk_norm=True,
                       shared_lm_head=True, rope_theta=5e5, z_loss_scale=1e-6),
    "Mixtral-8x7B": dict(num_layers=32, hidden_dim=4096, num_heads=32, num_kv_heads=8, num_experts=8,
                         moe_ffn_dim=14336, vocab_size=32768, num_groups=1),
}


def model_config(
    *,
    num_layers: int,
    hidden_dim: int,
    num_heads: int,
    num_kv_heads: Optional[int],
    num_experts: int,
    moe_ffn_dim: int,
    vocab_size: int,
    num_groups: int = 1,
    outer_batch: int = 1,
    rope_theta: float = 1e6,
    capacity_factor: float = 2.0,
    num_experts_per_token: int = 2,
    load_balance_loss_weight: float = 0.01,
    router_z_loss_weight: float = 0.0,
    ffn_layer_types: Sequence[str] = ("sparse",),
    dense_ffn_dim: Optional[int] = None,
    shared_lm_head: bool = False,
    stack_cfg: Optional[InstantiableConfig] = None,
    scan_chunk: Optional[int] = None,
    drop_free: bool = False,
    atten_hidden_dim: Optional[int] = None,
    qk_norm: bool = False,
    norm_eps: float = 1e-5,
    z_loss_scale: float = 0.0,
    ffn_structure: str = "prenorm",
) -> causal_lm.Model.Config:
    """RMSNorm / RoPE / SwiGLU decoder whose feed-forward layers follow ``ffn_layer_types``
    (cycled over the stack): "sparse" = MoE, "dense" = ordinary FFN.  ``drop_free`` selects the
    sorted grouped-GEMM experts with capacity-free top-k routing; ``atten_hidden_dim`` decouples
    the attention width (heads x head dim) from the model width; ``qk_norm`` adds per-head
    RMSNorm on queries and keys."""
    if num_kv_heads:
        atten_cfg = GroupedQueryAttention.default_config()
        input_linear = FusedGroupedQKVLinear.default_config().set(num_kv_heads=num_kv_heads)
    else:
        atten_cfg = MultiheadAttention.default_config()
        input_linear = FusedQKVLinear.default_config()
    qkv = RoFormerQKVLinear.default_config().set(input_linear=input_linear, rotary_value=False)
    qkv.rope_pos_emb_layer.theta = rope_theta
    if atten_hidden_dim is not None:
        atten_cfg.hidden_dim = atten_hidden_dim
    if qk_norm:
        head_norm = RMSNorm.default_config().set(eps=norm_eps, forward_dtype=None)
        atten_cfg.query_scale.norm = head_norm
        atten_cfg.key_scale.norm = head_norm.clone()
    if drop_free:
        gating = TopKDropFreeGating.default_config().set(num_experts_per_token=num_experts_per_token)
    elif num_experts_per_token == 2:
        gating = Top2Gating.default_config().set(
            train_capacity_factor=capacity_factor, eval_capacity_factor=capacity_factor)
    else:
        gating = TopKGating.default_config().set(
            num_experts_per_token=num_experts_per_token, train_capacity_factor=capacity_factor,
            eval_capacity_factor=capacity_factor)
    moe_cls = TransformerFeedForwardDropFreeMoE if drop_free else TransformerFeedForwardMoE
    expert_cfg = moe_cls.default_config().set(
        num_experts=num_experts, num_groups=num_groups, outer_batch=outer_batch, gating=gating,
        load_balance_loss_weight=load_balance_loss_weight, router_z_loss_weight=router_z_loss_weight)
    cfg = common_model_config(
        num_layers=num_layers, hidden_dim=hidden_dim, num_heads=num_heads, vocab_size=vocab_size,
        stack_cfg=stack_cfg if stack_cfg is not None else RepeatedTransformerLayer.default_config(),
        activation_fn=("nn.silu", "linear"), ffn_dim=dense_ffn_dim or moe_ffn_dim,
        normalization=RMSNorm.default_config().set(eps=norm_eps, forward_dtype=None),
        emb_cfg=TransformerTextEmbeddings.default_config().set(pos_emb=None),
        lm_head_cfg=LmHead.default_config() if not shared_lm_head else None,
        attention_cfg=atten_cfg, attention_qkv_linear=qkv, ffn_layer_types=tuple(ffn_layer_types),
        expert_cfg=expert_cfg, moe_ffn_dim=moe_ffn_dim, scan_chunk=scan_chunk, ffn_structure=ffn_structure)
    cfg.aux_loss_regex = ".*/aux_loss"
    cfg.metrics = causal_lm.metrics_config(aux_loss_regex=cfg.aux_loss_regex, z_loss_scale=z_loss_scale)
    return cfg


def preset(name: str, **overrides) -> causal_lm.Model.Config:
    return model_config(**{**MODEL_PRESETS[name], **overrides})


def trainer_configs() -> dict:
    """Named MoE trainer configs: ``envy-{preset}`` (synthetic input unless a source is wired)."""
    from axlearn_b200.experiments.text.gpt.common import (
        MESH_AXIS_NAMES,
        adamw_decoupled_learner_config,
        get_trainer_config_fn,
        mesh_shape_from_axes,
    )

    def make(name):
        def fn():
            mk = dict(MODEL_PRESETS[name])
            small = name == "test"
            switch = name.startswith("Switch")
            max_step = 50 if small else 250_000
            seq = 64 if small else (8192 if switch else 4096)
            if switch:
                # The reference's recipe for these sizes: decoupled AdamW at 1e-2 with mup-simple
                # scaling of the matrix updates (base width 768), decay to 0.5 %, 8M tokens / batch.
                from axlearn_b200.experiments.text.gpt.common import mup_simple_adam_update_transformation

                learner = adamw_decoupled_learner_config(
                    peak_lr=0.01, max_step=max_step, weight_decay=1e-4, lr_warmup_steps=5000, alpha=0.005,
                    adam_update_transformation=mup_simple_adam_update_transformation(768 / mk["hidden_dim"]))
                batch = 8 * 2 ** 20 // seq
                mesh = mesh_shape_from_axes(fsdp=-1, expert=16)
            else:
                learner = adamw_decoupled_learner_config(
                    peak_lr=3e-4 if not small else 3e-3, max_step=max_step, weight_decay=0.1,
                    lr_warmup_steps=2 if small else 2000)
                batch = 8 if small else 16
                mesh = mesh_shape_from_axes(expert=-1) if not small else mesh_shape_from_axes()
            return get_trainer_config_fn(
                model_cfg=model_config(scan_chunk=None if small else 8192, **mk), learner_cfg=learner,
                max_step=max_step, train_batch_size=batch, max_sequence_length=seq, vocab_size=mk["vocab_size"],
                mesh_shape=mesh, mesh_axis_names=MESH_AXIS_NAMES, keep_every_n_steps=5000 if switch else 50_000)()

        return fn

    return {f"envy-{name}": make(name) for name in MODEL_PRESETS}
