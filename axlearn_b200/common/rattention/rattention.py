"""RAttention: softmax attention inside a sliding window, linear attention for everything older.

Reference: axlearn/common/rattention/rattention.py (``ResidualLinearAttention`` :72, ``RAttention``
:473-821), axlearn/common/rattention/kernels/linear_attention_kernels.py (chunked kernels and the
linear-scan reference :610-700), kernels/utils.py (feature maps), utils.py (``GroupRMSNorm``).

A query at position ``t`` attends with softmax to keys ``t - w .. t`` and, through a recurrent
state, to every key at or before ``t - w - 1``: ``o_t = phi(q_t) H_t`` with
``H_t = H_0 + sum_{s <= t - w - 1} phi(k_s)^T v_s``.  The two outputs are RMS-normalised per head
and added.  The decode state is the window's keys / values plus one ``[heads, dk', dv]`` matrix,
whatever the sequence length.

The linear part is computed chunk by chunk: inside a chunk a masked ``(Q K^T) V`` product, across
chunks the running state -- two GEMM-shaped products per chunk instead of a token-by-token scan.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from axlearn_b200.common.attention import (
    MultiheadInputLinear,
    MultiheadOutputLinear,
    RoFormerSinusoidalPositionalEmbedding,
    apply_rotary_position_embeddings,
)
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Dropout
from axlearn_b200.common.param_init import constant_initializer

Tensor = torch.Tensor


def feature_map(x: Tensor, kind: str = "softmax") -> Tensor:
    """``softmax``: ``[softmax(x), softmax(-x)]`` over the head dim; ``relu``: ``[relu(x), relu(-x)]``.
    Both double the feature width and keep features non-negative."""
    xf = x.float()
    if kind == "softmax":
        return torch.cat([torch.softmax(xf, dim=-1), torch.softmax(-xf, dim=-1)], dim=-1)
    if kind == "relu":
        return torch.cat([F.relu(xf), F.relu(-xf)], dim=-1)
    raise ValueError(f"unknown feature map {kind}")


def _shift_right(x: Tensor, shift: int) -> Tensor:
    """Along time (dim 2): position ``t`` receives ``x[t - shift]``, the first ``shift`` are zero."""
    if x.shape[2] <= shift:
        return torch.zeros_like(x)
    return F.pad(x[:, :, : x.shape[2] - shift], (0, 0, shift, 0))


def residual_linear_attention_reference(q, k, v, h0, *, window_size: int, feat_map: str = "softmax"):
    """Token-by-token scan.  ``q, k [B, N, T, dk]``, ``v [B, N, T, dv]``, ``h0 [B, N, dk', dv]``."""
    q, k = feature_map(q, feat_map), feature_map(k, feat_map)
    k, v = _shift_right(k, window_size + 1), _shift_right(v.float(), window_size + 1)
    h = h0.float()
    out = []
    for t in range(q.shape[2]):
        h = h + k[:, :, t, :, None] * v[:, :, t, None, :]
        out.append(torch.einsum("bnk,bnkv->bnv", q[:, :, t], h))
    return torch.stack(out, dim=2), h


def residual_linear_attention(q, k, v, h0, *, window_size: int, feat_map: str = "softmax", chunk_size: int = 512):
    """Chunked form of the scan; returns ``(output [B, N, T, dv], final state)``."""
    q, k = feature_map(q, feat_map), feature_map(k, feat_map)
    k, v = _shift_right(k, window_size + 1), _shift_right(v.float(), window_size + 1)
    h = h0.float()
    t_total = q.shape[2]
    outs = []
    for lo in range(0, t_total, chunk_size):
        qc, kc, vc = q[:, :, lo:lo + chunk_size], k[:, :, lo:lo + chunk_size], v[:, :, lo:lo + chunk_size]
        c = qc.shape[2]
        causal = torch.tril(torch.ones(c, c, dtype=torch.bool, device=q.device))
        scores = torch.einsum("bntk,bnsk->bnts", qc, kc).masked_fill(~causal, 0.0)
        outs.append(torch.einsum("bntk,bnkv->bntv", qc, h) + torch.einsum("bnts,bnsv->bntv", scores, vc))
        h = h + torch.einsum("bnsk,bnsv->bnkv", kc, vc)
    return torch.cat(outs, dim=2), h


class GroupRMSNorm(BaseLayer):
    """RMS normalisation per head on ``[B, T, heads, head_dim]`` with a ``[heads, head_dim]`` scale."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_groups: Required[int] = REQUIRED
        eps: float = 1e-8

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"scale": ParameterSpec(shape=(cfg.num_groups, cfg.input_dim), mesh_axes=(None, None),
                                       initializer=constant_initializer(1.0))}

    def forward(self, x: Tensor) -> Tensor:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self._config.eps)
        return (y * self.parameters["scale"].float()).to(x.dtype)


class RAttention(BaseLayer):
    """Self-attention layer: ``forward(query [B, T, D]) -> [B, T, D]``; ``init_states`` /
    ``extend_step`` decode one token at a time with a constant-size state."""

    @config_class
    class Config(BaseLayer.Config):
        query_dim: Required[int] = REQUIRED
        num_heads: Required[int] = REQUIRED
        sliding_window_size: int = 1024
        use_residual_la: bool = True
        feat_fn: str = "softmax"
        chunk_size: int = 512
        rope_theta: float = 500000.0
        use_qk_scale: bool = False                 # learned per-dimension scales on q / k of the linear branch
        dropout: InstantiableConfig = Dropout.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.query_dim % cfg.num_heads:
            raise ValueError("query_dim must be divisible by num_heads")
        h = cfg.query_dim // cfg.num_heads
        self._h = h
        for name in ("q_proj", "k_proj", "v_proj"):
            self._add_child(name, MultiheadInputLinear.default_config().set(
                model_dim=cfg.query_dim, num_heads=cfg.num_heads, per_head_dim=h, bias=False))
        self._add_child("o_proj", MultiheadOutputLinear.default_config().set(
            model_dim=cfg.query_dim, num_heads=cfg.num_heads, per_head_dim=h, bias=False))
        self._add_child("rope", RoFormerSinusoidalPositionalEmbedding.default_config().set(dim=h, theta=cfg.rope_theta))
        self._add_child("dropout", cfg.dropout)
        if cfg.use_residual_la:
            for name in ("swa_norm", "rla_norm"):
                self._add_child(name, GroupRMSNorm.default_config().set(input_dim=h, num_groups=cfg.num_heads))

    def _create_layer_parameter_specs(self):
        cfg = self._config
        if not (cfg.use_residual_la and cfg.use_qk_scale):
            return {}
        return {n: ParameterSpec(shape=(self._h,), mesh_axes=(None,), initializer=constant_initializer(1.0))
                for n in ("q_scale", "k_scale")}

    # ------------------------------------------------------------------ pieces
    def _project(self, x: Tensor, positions: Tensor):
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        sin = self.rope(positions=positions)[:, :, None, :]
        q_rot, k_rot, _ = apply_rotary_position_embeddings(query=q, key=k, value=v, sinusoidal_pos=sin)
        return q, k, v, q_rot, k_rot

    def _linear_inputs(self, q: Tensor, k: Tensor):
        """The linear branch sees un-rotated projections (optionally rescaled), heads first."""
        if self._config.use_qk_scale:
            q, k = q * self.parameters["q_scale"].to(q.dtype), k * self.parameters["k_scale"].to(k.dtype)
        return q.transpose(1, 2), k.transpose(1, 2)

    def _window_attention(self, q: Tensor, k: Tensor, v: Tensor, q_pos: Tensor, k_pos: Tensor, k_live=None) -> Tensor:
        w = self._config.sliding_window_size
        rel = q_pos[:, :, None] - k_pos[:, None, :]
        ok = (rel >= 0) & (rel <= w)
        if k_live is not None:
            ok = ok & k_live[:, None, :]
        logits = torch.einsum("btnh,bsnh->bnts", q.float(), k.float()) * self._h ** -0.5
        logits = logits.masked_fill(~ok[:, None], -1e30)
        probs = self.dropout(torch.softmax(logits, dim=-1))
        return torch.einsum("bnts,bsnh->btnh", probs, v.float())

    def _mix(self, swa: Tensor, rla: Optional[Tensor]) -> Tensor:
        if rla is None:
            return swa
        return self.swa_norm(swa) + self.rla_norm(rla.transpose(1, 2))

    # ------------------------------------------------------------------ training / prefill
    def forward(self, query: Tensor, *, positions: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        b, t, _ = query.shape
        if positions is None:
            positions = torch.arange(t, device=query.device)[None].expand(b, -1)
        q, k, v, q_rot, k_rot = self._project(query, positions)
        swa = self._window_attention(q_rot, k_rot, v, positions, positions)
        rla = None
        if cfg.use_residual_la:
            ql, kl = self._linear_inputs(q, k)
            h0 = query.new_zeros(b, cfg.num_heads, 2 * self._h, self._h, dtype=torch.float32)
            rla, _ = residual_linear_attention(ql, kl, v.transpose(1, 2), h0, window_size=cfg.sliding_window_size,
                                               feat_map=cfg.feat_fn, chunk_size=cfg.chunk_size)
        return self.o_proj(self._mix(swa, rla).to(query.dtype))

    # ------------------------------------------------------------------ decoding
    def init_states(self, *, batch_size: int, device=None, dtype=torch.float32) -> dict:
        """A ring of the last ``window + 1`` raw keys / values (with their positions) and the linear
        state of everything that has left the ring."""
        cfg = self._config
        w1 = cfg.sliding_window_size + 1
        z = lambda *s: torch.zeros(*s, device=device, dtype=dtype)
        return {"k": z(batch_size, w1, cfg.num_heads, self._h), "v": z(batch_size, w1, cfg.num_heads, self._h),
                "pos": torch.full((batch_size, w1), -1, dtype=torch.long, device=device),
                "h": torch.zeros(batch_size, cfg.num_heads, 2 * self._h, self._h, device=device),
                "time_step": torch.zeros(batch_size, dtype=torch.long, device=device)}

    def extend_step(self, *, cached_states: dict, query: Tensor):
        """``query [B, 1, D]`` at position ``time_step``; returns ``(states, [B, 1, D])``."""
        cfg = self._config
        st = cached_states
        t = st["time_step"]
        b = query.shape[0]
        rows = torch.arange(b, device=query.device)
        q, k, v, q_rot, _ = self._project(query, t[:, None])
        slot = t % (cfg.sliding_window_size + 1)
        h = st["h"]
        if cfg.use_residual_la:
            # The entry about to be overwritten is exactly window + 1 old: it joins the linear state.
            old_live = (st["pos"][rows, slot] >= 0).float()[:, None, None, None]
            _, old_k = self._linear_inputs(q, st["k"][rows, slot][:, None])
            phi_k = feature_map(old_k[:, :, 0], cfg.feat_fn)                           # [B, N, 2h]
            h = h + old_live * phi_k[..., :, None] * st["v"][rows, slot].float()[..., None, :]
        new_k, new_v, new_pos = st["k"].clone(), st["v"].clone(), st["pos"].clone()
        new_k[rows, slot], new_v[rows, slot], new_pos[rows, slot] = k[:, 0].to(new_k.dtype), v[:, 0].to(new_v.dtype), t
        live = new_pos >= 0
        sin = self.rope(positions=new_pos.clamp_min(0))[:, :, None, :]
        _, k_rot, _ = apply_rotary_position_embeddings(query=new_k, key=new_k, value=new_v, sinusoidal_pos=sin)
        swa = self._window_attention(q_rot, k_rot, new_v, t[:, None], new_pos, k_live=live)
        rla = None
        if cfg.use_residual_la:
            ql, _ = self._linear_inputs(q, k)
            rla = torch.einsum("bnk,bnkv->bnv", feature_map(ql[:, :, 0], cfg.feat_fn), h)[:, :, None]
        out = self.o_proj(self._mix(swa, rla).to(query.dtype))
        return {"k": new_k, "v": new_v, "pos": new_pos, "h": h, "time_step": t + 1}, out
