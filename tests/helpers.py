"""Shared builders for tests."""

import torch

from axlearn_b200.experiments.text.gpt import fuji
from axlearn_b200.experiments.text.gpt.common import (
    adamw_decoupled_learner_config,
    get_trainer_config_fn,
    mesh_shape_from_axes,
)


def tiny_fuji_trainer_config(directory, *, max_step=20, save_every_n_steps=10, stack_cfg=None,
                             train_dtype=None, device="cpu", num_kv_heads=None, shared_lm_head=False,
                             mesh_shape=None, batch=8, seq=64, scan_chunk=None, hidden=128, layers=4,
                             heads=4, ffn=512, vocab=32768):
    """The smallest benchmark config: 4 layers, d_model 128, 4 heads, SwiGLU 512, RMSNorm eps 1e-5, RoPE
    theta 5e5, vocab 32768, untied head, batch 8 x seq 64, AdamW lr 3e-4 b1 .9 b2 .95 wd .1."""
    model = fuji.model_config(
        num_layers=layers, hidden_dim=hidden, num_heads=heads, num_kv_heads=num_kv_heads, vocab_size=vocab,
        rope_theta=5e5, shared_lm_head=shared_lm_head, ffn_dim=ffn, stack_cfg=stack_cfg, scan_chunk=scan_chunk)
    learner = adamw_decoupled_learner_config(peak_lr=3e-4, max_step=max_step, weight_decay=0.1, lr_warmup_steps=2)
    cfg = get_trainer_config_fn(
        model_cfg=model, learner_cfg=learner, max_step=max_step, train_batch_size=batch,
        max_sequence_length=seq, vocab_size=vocab, mesh_shape=mesh_shape or mesh_shape_from_axes(),
        train_dtype=train_dtype, save_every_n_steps=save_every_n_steps)()
    cfg.dir = str(directory)
    cfg.device = device
    return cfg


def to_plain(obj):
    """Tensors -> numpy arrays, recursively: values put on a multiprocessing queue must not
    depend on the sending process staying alive (torch shares tensor storage by file descriptor,
    which fails when the sender has exited before the receiver unpickles)."""
    import torch

    if isinstance(obj, torch.Tensor):
        return ("__tensor__", obj.detach().cpu().float().numpy() if obj.dtype == torch.bfloat16 else obj.detach().cpu().numpy(),
                str(obj.dtype))
    if isinstance(obj, dict):
        return {k: to_plain(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(to_plain(v) for v in obj)
    return obj


def from_plain(obj):
    import torch

    if isinstance(obj, tuple) and len(obj) == 3 and obj[0] == "__tensor__":
        t = torch.from_numpy(obj[1])
        return t.bfloat16() if obj[2] == "torch.bfloat16" else t
    if isinstance(obj, dict):
        return {k: from_plain(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(from_plain(v) for v in obj)
    return obj
