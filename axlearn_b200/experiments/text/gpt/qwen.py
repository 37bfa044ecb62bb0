"""Qwen3-style mixture-of-experts decoders (drop-free top-k routing over many small experts).

Parity target in the reference: axlearn/experiments/text/gpt/qwen.py:60-260 -- ``30B-A3B``: 48
layers, model width 2048, attention width 32 x 128 = 4096 with 4 KV heads and per-head RMSNorm on
queries and keys, 128 SwiGLU experts of hidden 768 with 8 active per token and no capacity limit
(``TransformerFeedForwardDropFreeMoE``), untied LM head, vocabulary 151936, RMSNorm eps 1e-6, RoPE
theta 1e6, z-loss 1e-6; default mesh ``fsdp=8, data=-1``.
"""

from __future__ import annotations

from axlearn_b200.common import causal_lm
from axlearn_b200.experiments.text.gpt import envy

QWEN3_VOCAB_SIZE = 151936
QWEN3_BOS_TOKEN_ID = 151643
QWEN3_EOS_TOKEN_ID = 151645
QWEN3_PAD_TOKEN_ID = 151645
QWEN3_RMS_NORM_EPS = 1e-6
QWEN3_ROPE_THETA = 1_000_000.0
QWEN3_HEAD_DIM = 128

MODEL_PRESETS = {
    "test": dict(num_layers=2, hidden_dim=64, num_heads=4, num_kv_heads=2, atten_hidden_dim=128,
                 num_experts=8, moe_ffn_dim=64, num_experts_per_token=2, vocab_size=512),
    "30B-A3B": dict(num_layers=48, hidden_dim=16 * 128, num_heads=32, num_kv_heads=4,
                    atten_hidden_dim=32 * QWEN3_HEAD_DIM, num_experts=128, moe_ffn_dim=768,
                    num_experts_per_token=8, vocab_size=QWEN3_VOCAB_SIZE),
}


def model_config(**kwargs) -> causal_lm.Model.Config:
    defaults = dict(drop_free=True, qk_norm=True, norm_eps=QWEN3_RMS_NORM_EPS, rope_theta=QWEN3_ROPE_THETA,
                    z_loss_scale=1e-6, shared_lm_head=False, ffn_layer_types=("sparse",), num_groups=1,
                    load_balance_loss_weight=1e-3)
    return envy.model_config(**{**defaults, **kwargs})


def preset(name: str, **overrides) -> causal_lm.Model.Config:
    return model_config(**{**MODEL_PRESETS[name], **overrides})


# (tokens per batch, sequence length) variants of every size, as in the reference.
CONFIGS = {"30B-A3B": [(8 * 1024 * 1024, 8 * 1024), (16 * 1024 * 1024, 32 * 1024)]}


def trainer_configs() -> dict:
    """``qwen3-{size}-bs{tokens per batch}m-seq{length}k`` trainer configs plus ``qwen3-test``
    (synthetic input unless a source is wired).  Learner: decoupled AdamW at 1e-2 decaying to
    0.5 %, weight decay 1e-4, 5000 warm-up steps."""
    from axlearn_b200.experiments.text.gpt.common import (
        MESH_AXIS_NAMES,
        adamw_decoupled_learner_config,
        get_trainer_config_fn,
        mesh_shape_from_axes,
    )

    def make(size, tokens_per_batch=None, seq_len=None):
        def fn():
            mk = dict(MODEL_PRESETS[size])
            small = size == "test"
            max_step = 50 if small else 250_000
            return get_trainer_config_fn(
                model_cfg=model_config(scan_chunk=None if small else 8192, **mk),
                learner_cfg=adamw_decoupled_learner_config(
                    peak_lr=3e-3 if small else 0.01, max_step=max_step, weight_decay=1e-4, alpha=1 / 200.0,
                    lr_warmup_steps=2 if small else 5000),
                max_step=max_step, train_batch_size=8 if small else tokens_per_batch // seq_len,
                max_sequence_length=64 if small else seq_len, vocab_size=mk["vocab_size"],
                mesh_shape=mesh_shape_from_axes() if small else mesh_shape_from_axes(fsdp=8, data=-1),
                mesh_axis_names=MESH_AXIS_NAMES, keep_every_n_steps=5000, eval_every_n_steps=25_000)()

        return fn

    out = {"qwen3-test": make("test")}
    for size, variants in CONFIGS.items():
        for tokens, seq in variants:
            out[f"qwen3-{size}-bs{tokens // 1024 // 1024}m-seq{seq // 1024}k"] = make(size, tokens, seq)
    return out
