"""Mixture-of-experts feed-forward layers with capacity-based top-k routing.

Parity targets in the reference (axlearn/common/mixture_of_experts.py): ``_router_z_loss`` (:158),
``_compute_expert_capacity`` (:224), ``AdaptiveLoadBalanceLoss`` (:307), ``BaseGating`` (:365),
``Top2Gating`` (:461-725), ``TopKGating`` (:727-1098) and ``TransformerFeedForwardMoE`` (:1443-1800),
including the routing semantics: tokens are grouped ``[outer_batch, groups, group_size]``; within
a group experts fill up in priority order (every token's first choice before any second choice,
tokens in sequence order), assignments beyond ``expert_capacity`` are dropped, gate weights are
renormalised over the chosen experts, and the load-balance loss is
``mean(density * density_proxy) * E^2`` (``/ k`` for top-k).

Representation.  The reference materialises one-hot ``[O, G, S, E, C]`` dispatch / combine
tensors and moves tokens with einsums.  Here routing is kept as indices -- for every
(token, choice): expert id, slot in that expert's buffer (or "dropped") and weight -- and tokens
move by gather / scatter (``dispatch`` / ``combine``), which is O(tokens * k * model_dim) memory
traffic instead of O(tokens * E * C).  The dense tensors are still available
(``Routing.combine_tensor()`` / ``dispatch_tensor()``) for parity checks.

Expert parallelism.  Expert weights are sharded over the ``expert`` mesh axis on their leading
dim (marked ``ComputeAxis``: never gathered).  Each rank routes its own tokens, an all-to-all
over the ``expert`` axis brings every expert the tokens of all ranks, the expert FFN runs as
per-expert GEMMs, and a second all-to-all returns the outputs to the ranks that own the tokens.
"""

from __future__ import annotations

import dataclasses
import math
from typing import Any, Optional, Sequence, Union

import torch

from axlearn_b200 import ops
from axlearn_b200.common.base_layer import BaseLayer, FanAxes, ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Dropout, LayerNorm, StochasticDepth, get_activation_fn
from axlearn_b200.common.module import Module, nowrap
from axlearn_b200.common.param_init import constant_initializer
from axlearn_b200.parallel import collectives as coll
from axlearn_b200.parallel.mesh import current_mesh

Tensor = torch.Tensor


def _router_z_loss(logits: Tensor) -> Tensor:
    """``mean(logsumexp(logits)^2)``: keeps router logits small."""
    return torch.logsumexp(logits.float(), dim=-1).square().mean()


def _cap_logits(logits: Tensor, cap: float) -> Tensor:
    return cap * torch.tanh(logits / cap) if cap > 0 else logits


def _compute_expert_capacity(*, group_size: int, num_experts: int, expert_capacity: Optional[int],
                             capacity_factor: Optional[float]) -> int:
    if not (capacity_factor or expert_capacity):
        raise ValueError("At least one of `capacity_factor` or `expert_capacity` needs to be set.")
    if capacity_factor:
        auto = int(group_size * capacity_factor / num_experts)
        if expert_capacity is None:
            expert_capacity = 1
        expert_capacity = max(expert_capacity, auto)
    return expert_capacity


@dataclasses.dataclass
class Routing:
    """Index form of a routing decision for tokens ``[O, G, S]`` and ``K`` choices each."""

    expert_index: Tensor   # int64 [O, G, S, K]
    slot: Tensor           # int64 [O, G, S, K]: position in the expert's buffer, -1 = dropped
    weight: Tensor         # float32 [O, G, S, K]: combine weight (0 for dropped assignments)
    num_experts: int
    expert_capacity: int
    load_balance_loss: Optional[Tensor] = None
    router_z_loss: Optional[Tensor] = None

    def dispatch_tensor(self) -> Tensor:
        """Dense bool ``[O, G, S, E, C]`` (the reference's representation)."""
        return self.combine_tensor(weights=False) > 0

    def combine_tensor(self, weights: bool = True) -> Tensor:
        o, g, s, k = self.expert_index.shape
        out = torch.zeros((o, g, s, self.num_experts * self.expert_capacity + 1), dtype=torch.float32,
                          device=self.expert_index.device)
        flat = torch.where(self.slot >= 0, self.expert_index * self.expert_capacity + self.slot,
                           torch.full_like(self.slot, self.num_experts * self.expert_capacity))
        vals = self.weight if weights else (self.slot >= 0).float()
        out.scatter_add_(3, flat, vals)
        return out[..., :-1].reshape(o, g, s, self.num_experts, self.expert_capacity)


def _slots_in_priority_order(expert_index: Tensor, num_experts: int, capacity: int) -> Tensor:
    """Position of each (token, choice) in its expert's buffer: all first choices in sequence
    order, then all second choices, ...; -1 where the expert is already full.

    One stable sort of the (group, expert) keys in choice-major order: the rank of an entry
    among equal keys is its position (the reference takes a cumulative sum over a one-hot
    ``[.., K*S, E]`` tensor instead)."""
    o, g, s, k = expert_index.shape
    flat = expert_index.permute(0, 1, 3, 2).reshape(o * g, k * s)           # choice-major
    group = torch.arange(o * g, device=flat.device)[:, None]
    keys = (group * num_experts + flat).reshape(-1)
    order = torch.sort(keys, stable=True).indices
    counts = torch.bincount(keys, minlength=o * g * num_experts)
    starts = counts.cumsum(0) - counts
    ranks = torch.arange(keys.numel(), device=keys.device) - starts[keys[order]]
    pos = torch.empty_like(keys)
    pos[order] = ranks
    pos = torch.where(pos < capacity, pos, torch.full_like(pos, -1))
    return pos.reshape(o, g, k, s).permute(0, 1, 3, 2).contiguous()


def _expert_counts(index: Tensor, num_experts: int) -> Tensor:
    """``index [O, G, S]`` of expert ids -> how many tokens chose each expert ``[O, G, E]``."""
    o, g, s = index.shape
    group = torch.arange(o * g, device=index.device)[:, None]
    keys = (group * num_experts + index.reshape(o * g, s)).reshape(-1)
    return torch.bincount(keys, minlength=o * g * num_experts).reshape(o, g, num_experts)


class AdaptiveLoadBalanceLoss(BaseLayer):
    """Scales the load-balance loss up (down) when the moving average of the over-capacity
    ratio is above ``max_value`` (below ``min_value``); the scale lives in log space."""

    @config_class
    class Config(BaseLayer.Config):
        moving_average_weight: float = 0.99
        max_value: Required[float] = REQUIRED
        min_value: float = 1e-3
        log_step: float = 0.01

    def _create_layer_parameter_specs(self):
        zero = constant_initializer(0.0)
        return {
            "value_average": ParameterSpec(shape=(), dtype=torch.float32, initializer=zero, weight_decay_scale=0.0),
            "log_scale": ParameterSpec(shape=(), dtype=torch.float32, initializer=zero, weight_decay_scale=0.0),
        }

    def forward(self, value: Tensor) -> Tensor:
        cfg = self._config
        avg = self.parameters["value_average"].detach()
        log_scale = self.parameters["log_scale"].detach()
        new_avg = cfg.moving_average_weight * avg + (1 - cfg.moving_average_weight) * value.detach().float()
        inc = (new_avg > cfg.max_value).float() - (new_avg < cfg.min_value).float()
        new_log_scale = log_scale + inc * cfg.log_step
        self.add_state_update("value_average", new_avg)
        self.add_state_update("log_scale", new_log_scale)
        self.add_summary("value_average", new_avg)
        self.add_summary("log_scale", new_log_scale)
        return torch.exp(new_log_scale)


class BaseGating(BaseLayer):
    """Turns router logits ``[O, G, S, E]`` into a ``Routing``."""

    @config_class
    class Config(BaseLayer.Config):
        num_experts: Required[int] = REQUIRED

    Output = Routing

    def forward(self, logits: Tensor) -> Routing:
        raise NotImplementedError(type(self))

    @nowrap
    def dispatch(self, x: Tensor, routing: Routing) -> Tensor:
        """``x [O, G, S, M] -> [O, E, G, C, M]``: every kept (token, choice) lands in its
        expert's slot; unfilled slots are zero."""
        from axlearn_b200.ops import moe_ops

        o, g, s, m = x.shape
        e, c = routing.num_experts, routing.expert_capacity
        out = moe_ops.dispatch(x.reshape(o * g * s, m), _flat_destinations(routing), o * e * g * c)
        return out.reshape(o, e, g, c, m)

    @nowrap
    def combine(self, y: Tensor, routing: Routing, *, dtype=None) -> Tensor:
        """``y [O, E, G, C, M] -> [O, G, S, M]``: weighted sum of each token's expert outputs."""
        from axlearn_b200.ops import moe_ops

        o, e, g, c, m = y.shape
        s, k = routing.expert_index.shape[2:]
        out = moe_ops.combine(y.reshape(o * e * g * c, m), routing.weight.reshape(o * g * s, k),
                              _flat_destinations(routing))
        return out.reshape(o, g, s, m).to(dtype or y.dtype)


def _flat_destinations(routing: Routing) -> Tensor:
    """``[T, K]``: row of the flattened ``[O, E, G, C]`` expert buffer for every (token, choice),
    -1 for dropped assignments."""
    o, g, s, k = routing.expert_index.shape
    e, c = routing.num_experts, routing.expert_capacity
    dev = routing.expert_index.device
    oo = torch.arange(o, device=dev).view(o, 1, 1, 1)
    gg = torch.arange(g, device=dev).view(1, g, 1, 1)
    dest = ((oo * e + routing.expert_index) * g + gg) * c + routing.slot
    return torch.where(routing.slot >= 0, dest, torch.full_like(dest, -1)).reshape(o * g * s, k)


def _fused_routing_ok(layer, logits: Tensor, k: int) -> bool:
    """The routing kernel covers plain top-k selection (subclasses that pick experts differently
    keep the step-by-step path)."""
    from axlearn_b200.ops import moe_ops

    default_index = type(layer)._compute_index in (Top2Gating._compute_index, TopKGating._compute_index)
    return default_index and moe_ops.gate_kernel_ok(logits, k)


def _fused_routing(layer, logits: Tensor, *, k: int, capacity: int):
    """``(index, gates, slot [O,G,S,K], counts [O,G,K,E], score_sums [O,G,E], lse [O,G,S])`` from
    the routing kernel, or None when it does not apply.  ``logits`` are already capped."""
    if not _fused_routing_ok(layer, logits, k):
        return None
    from axlearn_b200.ops import moe_ops

    o, g, s, e = logits.shape
    index, gates, slot, counts, sums, lse = moe_ops.topk_gate(logits.reshape(o * g, s, e), k, capacity)
    return (index.reshape(o, g, s, k), gates.reshape(o, g, s, k), slot.reshape(o, g, s, k),
            counts.reshape(o, g, k, e), sums.reshape(o, g, e), lse.reshape(o, g, s))


class Top2Gating(BaseGating):
    """Top-2 routing with capacity (GShard).  The second choice is the best expert other than
    the first; gate weights are renormalised over the two."""

    @config_class
    class Config(BaseGating.Config):
        gating_logit_cap: float = 0.0
        train_capacity_factor: float = 2.0
        eval_capacity_factor: float = 2.0
        expert_capacity: Optional[int] = None
        adaptive_load_balance_loss: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.adaptive_load_balance_loss is not None:
            self._add_child("adaptive_load_balance_loss", cfg.adaptive_load_balance_loss)

    def _compute_index(self, raw_gates: Tensor, *, k: int) -> Tensor:
        return raw_gates.topk(k, dim=-1).indices

    def forward(self, logits: Tensor) -> Routing:
        cfg = self._config
        logits = _cap_logits(logits.float(), cfg.gating_logit_cap)
        e = cfg.num_experts
        capacity = _compute_expert_capacity(
            expert_capacity=cfg.expert_capacity,
            capacity_factor=cfg.train_capacity_factor if self.is_training else cfg.eval_capacity_factor,
            group_size=logits.shape[-2], num_experts=e)
        raw_gates = None if _fused_routing_ok(self, logits, 2) else torch.softmax(logits, dim=-1)
        fused = _fused_routing(self, logits, k=2, capacity=capacity)
        if fused is not None:
            # One routing kernel: scores, top-2, capacity positions, per-expert counts and score sums.
            index, gates, slot, counts, score_sums, lse = fused
            weights = gates / (gates.sum(dim=-1, keepdim=True) + 1e-9)
            first, second = counts[:, :, 0], counts[:, :, 1]
            density_proxy = score_sums / index.shape[2]
            z = lse.square().mean()
        else:
            index = self._compute_index(raw_gates, k=2)                          # [O, G, S, 2]
            gate_1 = torch.gather(raw_gates, -1, index[..., :1]).squeeze(-1)
            gate_2 = torch.gather(raw_gates, -1, index[..., 1:]).squeeze(-1)
            gate_2 = torch.where(index[..., 0] == index[..., 1], torch.zeros_like(gate_2), gate_2)
            denom = gate_1 + gate_2 + 1e-9
            weights = torch.stack([gate_1 / denom, gate_2 / denom], dim=-1)
            first = _expert_counts(index[..., 0], e)                            # [O, G, E]
            second = _expert_counts(index[..., 1], e)
            density_proxy = raw_gates.mean(dim=-2)
            slot = _slots_in_priority_order(index, e, capacity)
            z = _router_z_loss(logits)
        # Load balance: fraction of tokens whose first choice is e, times the mean gate of e.
        density_1 = first.float() / index.shape[2]
        aux = (density_1 * density_proxy).mean() * e * e
        kept = slot >= 0
        weights = weights * kept.float()
        over_1 = (first - capacity).clamp(min=0).sum() / first.sum().clamp(min=1)
        second_total = second + first
        over_2 = (second_total - capacity).clamp(min=0).sum() / second_total.sum().clamp(min=1)
        counts = kept.sum(dim=-1)
        for i in range(3):
            self.add_summary(f"dispatch_{i}", (counts == i).sum())
        self.add_summary("router_z_loss", z.detach())
        self.add_summary("over_capacity_1", over_1)
        self.add_summary("over_capacity_2", over_2)
        if "adaptive_load_balance_loss" in self._children:
            self.add_summary("load_balance_loss_original", aux.detach())
            aux = aux * self.adaptive_load_balance_loss(torch.maximum(over_1, over_2))
        self.add_summary("load_balance_loss", aux.detach())
        self.add_module_output("gate_assignment", index)
        return Routing(expert_index=index, slot=slot, weight=weights, num_experts=e, expert_capacity=capacity,
                       load_balance_loss=aux, router_z_loss=z)


class TopKGating(BaseGating):
    """Top-k routing with capacity; weights are the raw gates renormalised over the k chosen
    experts (dropped assignments simply vanish from the sum)."""

    @config_class
    class Config(BaseGating.Config):
        num_experts_per_token: int = 2
        gating_logit_cap: float = 0.0
        train_capacity_factor: Optional[float] = None
        eval_capacity_factor: Optional[float] = None
        expert_capacity: Optional[int] = None
        adaptive_load_balance_loss: Optional[InstantiableConfig] = None
        noisy_gating: Optional[str] = None   # "gumbel"
        score_fn: Optional[Any] = None       # None = softmax; "sigmoid" or a callable(logits, dim)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.adaptive_load_balance_loss is not None:
            self._add_child("adaptive_load_balance_loss", cfg.adaptive_load_balance_loss)

    def _score(self, logits: Tensor) -> Tensor:
        fn = self._config.score_fn
        if fn is None:
            return torch.softmax(logits, dim=-1)
        if fn == "sigmoid":
            return torch.sigmoid(logits)
        return fn(logits, -1)

    def _compute_index(self, raw_gates: Tensor, *, k: int) -> Tensor:
        return raw_gates.topk(k, dim=-1).indices

    def _expert_capacity(self, group_size: int) -> int:
        cfg = self._config
        factor = cfg.train_capacity_factor if self.is_training else cfg.eval_capacity_factor
        if factor is None:
            factor = float(cfg.num_experts_per_token)
        return _compute_expert_capacity(expert_capacity=cfg.expert_capacity, capacity_factor=factor,
                                        group_size=group_size, num_experts=cfg.num_experts)

    def forward(self, logits: Tensor) -> Routing:
        cfg = self._config
        e, k = cfg.num_experts, cfg.num_experts_per_token
        logits = logits.float()
        self.add_summary("router_logit_rms", logits.detach().square().mean().sqrt())
        logits = _cap_logits(logits, cfg.gating_logit_cap)
        if cfg.noisy_gating is not None:
            if cfg.noisy_gating != "gumbel":
                raise NotImplementedError(cfg.noisy_gating)
            from axlearn_b200.common import prng

            u = prng.uniform(self.prng_key, logits.shape, device=logits.device).clamp(1e-20, 1.0)
            logits = logits - torch.log(-torch.log(u))
        capacity = self._expert_capacity(logits.shape[-2])
        fused = _fused_routing(self, logits, k=k, capacity=capacity) if cfg.score_fn is None else None
        if fused is not None:
            index, gate_w, slot, counts, score_sums, lse = fused
            z = lse.square().mean()
            totals = counts.sum(dim=2)                                        # [O, G, E]
            mean_scores = score_sums / index.shape[2]
        else:
            z = _router_z_loss(logits)
            raw_gates = self._score(logits)
            index = self._compute_index(raw_gates, k=k)
            gate_w = torch.gather(raw_gates, -1, index)
            normalized = raw_gates if cfg.score_fn is None else raw_gates / raw_gates.sum(dim=-1, keepdim=True)
            # top-k indices of a token are distinct, so "assigned" counts are plain counts.
            totals = sum(_expert_counts(index[..., j], e) for j in range(k))      # [O, G, E]
            mean_scores = normalized.mean(dim=-2)
            slot = _slots_in_priority_order(index, e, capacity)
        aux = (totals.float() / index.shape[2] * mean_scores).mean() * e * e / k
        kept = slot >= 0
        weights = gate_w / gate_w.sum(dim=-1, keepdim=True) * kept.float()
        over = (totals - capacity).clamp(min=0).sum() / totals.sum().clamp(min=1)
        self.add_summary("over_capacity_ratio", over)
        self.add_summary("router_z_loss", z.detach())
        counts = kept.sum(dim=-1)
        for i in range(k + 1):
            self.add_summary(f"dispatch_{i}", (counts == i).sum())
        if "adaptive_load_balance_loss" in self._children:
            self.add_summary("load_balance_loss_original", aux.detach())
            aux = aux * self.adaptive_load_balance_loss(over)
        self.add_summary("load_balance_loss", aux.detach())
        self.add_module_output("gate_assignment", index)
        return Routing(expert_index=index, slot=slot, weight=weights, num_experts=e, expert_capacity=capacity,
                       load_balance_loss=aux, router_z_loss=z)


class TransformerFeedForwardMoE(BaseLayer):
    """Drop-in replacement of the dense transformer feed-forward layer with ``num_experts``
    expert FFNs and a learned router (``gate_weight [M, E]``)."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        hidden_dim: Required[Union[int, InstantiableConfig]] = REQUIRED
        outer_batch: int = 1
        norm: InstantiableConfig = LayerNorm.default_config()
        activation: Union[str, tuple] = "nn.relu"
        dropout: InstantiableConfig = Dropout.default_config()
        stochastic_depth: InstantiableConfig = StochasticDepth.default_config()
        structure: str = "prenorm"
        residual_weight: float = 1.0
        num_experts: Required[int] = REQUIRED
        num_groups: Required[int] = REQUIRED
        gating: InstantiableConfig = Top2Gating.default_config()
        load_balance_loss_weight: float = 0.01
        router_z_loss_weight: float = 0.0
        # Logical dim name -> mesh axes, as in the reference ("e" = experts, "m" = model dim,
        # "h" = hidden dim).
        dim_to_mesh_axis_map: dict = {}

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.dim_to_mesh_axis_map = {
            "me": (None, None),
            "emh": (coll.ComputeAxis("expert"), None, "model"),
            "ehm": (coll.ComputeAxis("expert"), "model", None),
        }
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("gating", cfg.gating.clone(num_experts=cfg.num_experts))
        self._add_child("stochastic_depth", cfg.stochastic_depth)
        if cfg.structure in ("prenorm", "postnorm"):
            self._add_child("norm", cfg.norm.clone(input_dim=cfg.input_dim))
        elif cfg.structure == "hybridnorm":
            self._add_child("prenorm", cfg.norm.clone(input_dim=cfg.input_dim))
            self._add_child("postnorm", cfg.norm.clone(input_dim=cfg.input_dim))
        elif cfg.structure != "nonorm":
            raise NotImplementedError(cfg.structure)
        if cfg.structure in ("prenorm", "hybridnorm", "nonorm"):
            self._add_child("dropout1", cfg.dropout)
            self._add_child("dropout2", cfg.dropout)
        else:
            self._add_child("dropout", cfg.dropout)

    @nowrap
    def hidden_dim(self) -> int:
        cfg = self._config
        if isinstance(cfg.hidden_dim, int):
            return cfg.hidden_dim
        return cfg.hidden_dim.clone(input_dim=cfg.input_dim).instantiate()

    def _create_layer_parameter_specs(self):
        cfg = self._config
        h = self.hidden_dim()
        axes = cfg.dim_to_mesh_axis_map
        params = {
            "gate_weight": ParameterSpec(shape=(cfg.input_dim, cfg.num_experts), mesh_axes=axes.get("me")),
            "wo_weight": ParameterSpec(shape=(cfg.num_experts, h, cfg.input_dim), mesh_axes=axes.get("ehm"),
                                       fan_axes=FanAxes(in_axis=-2, out_axis=-1, batch_axis=0)),
        }
        names = [f"wi_{i}_weight" for i in range(len(cfg.activation))] if isinstance(cfg.activation, tuple) else ["wi_weight"]
        for n in names:
            params[n] = ParameterSpec(shape=(cfg.num_experts, cfg.input_dim, h), mesh_axes=axes.get("emh"),
                                      fan_axes=FanAxes(in_axis=-2, out_axis=-1, batch_axis=0))
        return params

    # ------------------------------------------------------------------ forward
    def forward(self, inputs: Tensor) -> Tensor:
        cfg = self._config
        s = cfg.structure
        if s == "prenorm":
            x = self._dispatch_and_combine(self.norm(inputs))
            x = self.stochastic_depth(self.dropout2(x))
            if cfg.residual_weight != 1:
                x = x * cfg.residual_weight
            return x + inputs
        if s == "postnorm":
            x = self.stochastic_depth(self.dropout(self._dispatch_and_combine(inputs)))
            if cfg.residual_weight != 1:
                x = x * cfg.residual_weight
            return self.norm(x + inputs)
        if s == "hybridnorm":
            x = self.postnorm(self._dispatch_and_combine(self.prenorm(inputs)))
            x = self.stochastic_depth(self.dropout2(x))
            if cfg.residual_weight != 1:
                x = x * cfg.residual_weight
            return x + inputs
        x = self.stochastic_depth(self.dropout2(self._dispatch_and_combine(inputs)))
        return x * cfg.residual_weight if cfg.residual_weight != 1 else x

    def _expert_weight(self, name: str, logical: str) -> Tensor:
        cfg = self._config
        spec = cfg.dim_to_mesh_axis_map.get(logical)
        w = self.parameters[name]
        shape = {"emh": (cfg.num_experts, cfg.input_dim, self.hidden_dim()),
                 "ehm": (cfg.num_experts, self.hidden_dim(), cfg.input_dim)}[logical]
        return coll.unshard_param(w, spec, compute_shape=coll.compute_shape(shape, spec))

    def _dispatch_and_combine(self, x: Tensor) -> Tensor:
        cfg = self._config
        in_dtype = x.dtype
        token_shape = x.shape[:-1]
        o = cfg.outer_batch
        if x.shape[0] % o:
            raise ValueError(f"batch_size {x.shape[0]} has to be divisible by outer_batch {o}.")
        tokens = math.prod(token_shape) // o
        if tokens % cfg.num_groups:
            raise ValueError(f"{tokens} tokens per outer batch must be divisible by num_groups({cfg.num_groups}).")
        x = x.reshape(o, cfg.num_groups, tokens // cfg.num_groups, cfg.input_dim)
        logits = torch.einsum("ogsm,me->ogse", x.float(), self.parameters["gate_weight"].float())
        routing = self.gating(logits)
        aux = routing.load_balance_loss * cfg.load_balance_loss_weight
        if cfg.router_z_loss_weight:
            aux = aux + routing.router_z_loss * cfg.router_z_loss_weight
        self.add_module_output("aux_loss", aux)
        fused = self._peer_exchange(x, routing)
        if fused is not None:
            return fused.to(in_dtype).reshape(*token_shape, cfg.input_dim)
        expert_in = self.gating.dispatch(x, routing)                          # [O, E, G, C, M]
        expert_out = self._experts(expert_in)
        out = self.gating.combine(expert_out, routing, dtype=in_dtype)
        return out.reshape(*token_shape, cfg.input_dim)

    def _expert_parallel_size(self) -> int:
        cfg = self._config
        mesh = current_mesh()
        ep = mesh.axis_size("expert") if mesh is not None and "expert" in mesh.shape else 1
        return ep if coll.has_axis((cfg.dim_to_mesh_axis_map.get("emh") or (None,))[0], "expert") else 1

    def _peer_exchange(self, x: Tensor, routing: Routing) -> Optional[Tensor]:
        """Expert parallelism over peer memory: token rows are stored straight into the memory of
        the GPU that owns their expert and expert outputs are read straight out of it, so the two
        all-to-alls are fused into the dispatch gather and the combine sum.  Returns None when the
        path does not apply (no expert axis, CPU / non-bf16 activations, more than 8 ranks)."""
        import os

        from axlearn_b200.ops import moe_ops

        cfg = self._config
        ep = self._expert_parallel_size()
        forced = os.environ.get("AXB_MOE_PEER_EXCHANGE") == "force"
        if not moe_ops.peer_exchange_ok(x) or ep > 8 or (ep == 1 and not forced):
            return None
        o, g, s, m = x.shape
        e, c = routing.num_experts, routing.expert_capacity
        k = routing.expert_index.shape[-1]
        slots = o * g * c
        dev = x.device
        oo = torch.arange(o, device=dev).view(o, 1, 1, 1)
        gg = torch.arange(g, device=dev).view(1, g, 1, 1)
        dest = routing.expert_index * slots + (oo * g + gg) * c + routing.slot   # expert-major rows
        dest = torch.where(routing.slot >= 0, dest, torch.full_like(dest, -1)).reshape(o * g * s, k)
        group = current_mesh().group("expert") if ep > 1 else None
        ex = moe_ops.expert_exchange(e // ep, slots, m, group, dev)
        xe = moe_ops.ep_dispatch(x.reshape(o * g * s, m), dest, ex)             # [E_local, ep * slots, M]
        ye = self._expert_ffn(xe)
        out = moe_ops.ep_combine(ye, routing.weight.reshape(o * g * s, k), dest, ex)
        return out.reshape(o, g, s, m)

    def _experts(self, x: Tensor) -> Tensor:
        """``[O, E, G, C, M] -> [O, E, G, C, M]`` through the expert FFNs, with the all-to-all
        pair around it when experts are sharded over the ``expert`` mesh axis."""
        cfg = self._config
        o, e, g, c, m = x.shape
        ep = self._expert_parallel_size()
        xe = x.permute(1, 0, 2, 3, 4).reshape(e, o * g * c, m)                # expert-major
        if ep > 1:
            # [E, T, M] -> every rank keeps E/ep experts and receives their tokens from all ranks.
            xe = coll.all_to_all(xe.reshape(ep, e // ep, o * g * c, m), "expert", split_dim=0, concat_dim=2)
            xe = xe.reshape(e // ep, ep * o * g * c, m)
        ye = self._expert_ffn(xe)
        if ep > 1:
            ye = ye.reshape(1, e // ep, ep, o * g * c, m)
            ye = coll.all_to_all(ye, "expert", split_dim=2, concat_dim=0).reshape(e, o * g * c, m)
        return ye.reshape(e, o, g, c, m).permute(1, 0, 2, 3, 4)

    def _expert_ffn(self, xe: Tensor) -> Tensor:
        """``[E_local, T, M]`` through each local expert's FFN (one GEMM per expert and
        projection; the tensor-parallel ``model`` split of the hidden dim is summed at the end)."""
        cfg = self._config
        act = cfg.activation
        outs = []
        wo = self._expert_weight("wo_weight", "ehm")
        if isinstance(act, tuple):
            wis = [self._expert_weight(f"wi_{i}_weight", "emh") for i in range(len(act))]
        else:
            wis = [self._expert_weight("wi_weight", "emh")]
        acts = list(act) if isinstance(act, tuple) else [act]
        x_in = coll.psum_grad(xe, "model") if coll.has_axis((cfg.dim_to_mesh_axis_map.get("emh") or (None,) * 3)[2], "model") else xe
        for i in range(xe.shape[0]):
            xi = x_in[i]
            hs = [ops.linear(xi, w[i].to(xi.dtype)) for w in wis]
            if len(hs) == 2 and acts == ["nn.silu", "linear"]:
                h = ops.swiglu(hs[0], hs[1])
            else:
                h = None
                for hv, a in zip(hs, acts):
                    hv = get_activation_fn(a)(hv)
                    h = hv if h is None else h * hv
            h = self.dropout1(h) if "dropout1" in self._children else h
            outs.append(ops.linear(h, wo[i].to(h.dtype)))
        y = torch.stack(outs, dim=0)
        if coll.has_axis((cfg.dim_to_mesh_axis_map.get("ehm") or (None,) * 3)[1], "model"):
            y = coll.psum(y, "model")
        return y


# ------------------------------------------------------------------------------------------
# Drop-free routing: every (token, choice) is served; experts see variable-length runs of rows.
# ------------------------------------------------------------------------------------------


@dataclasses.dataclass
class DropFreeRouting:
    gate_assignment: Tensor                 # [B, S, K] expert ids
    expert_weights: Tensor                  # [B, S, K] fp32, renormalised over the K choices
    load_balance_loss: Optional[Tensor] = None
    router_z_loss: Optional[Tensor] = None
    seq_load_balance_loss: Optional[Tensor] = None


class TopKDropFreeGating(TopKGating):
    """Top-k routing without capacity (reference: axlearn/common/mixture_of_experts.py:1101-1240):
    returns the chosen experts and their renormalised weights; the load-balance loss is
    ``mean(density * density_proxy) * E^2`` with the density counted over all K choices, and the
    optional per-sequence variant follows DeepSeek-V3 (eq. 17-20)."""

    def _normalized_gates(self, raw_gates: Tensor) -> Tensor:
        if self._config.score_fn is None:
            return raw_gates
        return raw_gates / raw_gates.sum(dim=-1, keepdim=True)

    def _load_balance_loss(self, raw_gates: Tensor, assignment: Tensor) -> Tensor:
        e = raw_gates.shape[-1]
        density = torch.bincount(assignment.reshape(-1), minlength=e).float() / assignment.numel()
        proxy = self._normalized_gates(raw_gates).reshape(-1, e).mean(dim=0)
        return (density * proxy).mean() * e * e

    def _seq_load_balance_loss(self, raw_gates: Tensor, assignment: Tensor) -> Tensor:
        b, s, e = raw_gates.shape
        k = assignment.shape[-1]
        one_hot_counts = torch.zeros((b, e), dtype=torch.float32, device=raw_gates.device)
        one_hot_counts.scatter_add_(1, assignment.reshape(b, -1), torch.ones((b, s * k), device=raw_gates.device))
        density = one_hot_counts * e / (s * k)
        proxy = self._normalized_gates(raw_gates).mean(dim=1)
        return (density * proxy).sum(dim=1).mean()

    def _process_logits(self, logits: Tensor) -> Tensor:
        cfg = self._config
        logits = _cap_logits(logits.float(), cfg.gating_logit_cap)
        if cfg.noisy_gating is not None:
            if cfg.noisy_gating != "gumbel":
                raise NotImplementedError(cfg.noisy_gating)
            from axlearn_b200.common import prng

            u = prng.uniform(self.prng_key, logits.shape, device=logits.device).clamp(1e-20, 1.0)
            logits = logits - torch.log(-torch.log(u))
        return logits

    def _select(self, raw_gates: Tensor, k: int) -> Tensor:
        return self._compute_index(raw_gates, k=k)

    def forward(self, logits: Tensor, seq_load_balance_loss_weight: Optional[float] = None) -> DropFreeRouting:
        cfg = self._config
        logits = self._process_logits(logits)                                   # [B, S, E]
        z = _router_z_loss(logits)
        self.add_summary("router_z_loss", z.detach())
        raw_gates = self._score(logits)
        assignment = self._select(raw_gates, cfg.num_experts_per_token)
        gate_w = torch.gather(raw_gates, -1, assignment)
        lb = self._load_balance_loss(raw_gates, assignment)
        self.add_summary("load_balance_loss", lb.detach())
        seq_lb = None
        if seq_load_balance_loss_weight:
            seq_lb = self._seq_load_balance_loss(raw_gates, assignment)
            self.add_summary("seq_load_balance_loss", seq_lb.detach())
        weights = gate_w / gate_w.sum(dim=-1, keepdim=True)
        self.add_module_output("gate_assignment", assignment)
        return DropFreeRouting(gate_assignment=assignment, expert_weights=weights, load_balance_loss=lb,
                               router_z_loss=z, seq_load_balance_loss=seq_lb)


class TopKBiasGating(TopKDropFreeGating):
    """Auxiliary-loss-free balancing (reference: :1243-1440, after DeepSeek-V3): a per-expert bias
    is added to the scores for *selection only* and nudged after every training step towards
    under-used experts (``+rate`` when an expert got fewer tokens than average, ``-rate`` when
    more); chosen weights are scaled by ``routed_scaling_factor``.  With ``num_group_of_experts >
    1`` only the ``topk_group`` best groups (by the sum of each group's two best adjusted scores)
    are eligible."""

    @config_class
    class Config(TopKDropFreeGating.Config):
        gating_update_rate: float = 1e-3
        routed_scaling_factor: float = 2.5
        num_group_of_experts: int = 1
        topk_group: int = 1

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"gate_bias": ParameterSpec(shape=(cfg.num_experts,), dtype=torch.float32,
                                           initializer=constant_initializer(0.0))}

    def _select(self, raw_gates: Tensor, k: int) -> Tensor:
        cfg = self._config
        adjusted = raw_gates + self.parameters["gate_bias"].float().detach()
        g = cfg.num_group_of_experts
        if g > 1:
            b, s, e = adjusted.shape
            per_group = adjusted.reshape(b, s, g, e // g)
            group_score = per_group.topk(min(2, e // g), dim=-1).values.sum(dim=-1)      # [B, S, G]
            keep = torch.zeros_like(group_score, dtype=torch.bool)
            keep.scatter_(-1, group_score.topk(cfg.topk_group, dim=-1).indices, True)
            adjusted = per_group.masked_fill(~keep[..., None], float("-inf")).reshape(b, s, e)
        index = adjusted.topk(k, dim=-1).indices
        if self.is_training:
            counts = torch.bincount(index.reshape(-1), minlength=cfg.num_experts).float()
            delta = torch.sign(counts.mean() - counts)
            self.add_state_update("gate_bias", (self.parameters["gate_bias"].float()
                                                + cfg.gating_update_rate * delta).detach())
        return index

    def forward(self, logits: Tensor, seq_load_balance_loss_weight: Optional[float] = None) -> DropFreeRouting:
        out = super().forward(logits, seq_load_balance_loss_weight)
        out.expert_weights = out.expert_weights * self._config.routed_scaling_factor
        return out


class TransformerFeedForwardDropFreeMoE(TransformerFeedForwardMoE):
    """Mixture of experts without token dropping (reference: :2321-2751).

    The (token, choice) pairs are sorted by expert -- choice-major, so that every token's first
    choice precedes any second choice inside an expert's run, as in the reference -- and laid
    out in one ``[R, M]`` buffer in which each expert's run starts on a block boundary (256 rows).  The
    three projections are then grouped GEMMs over that buffer (one tcgen05 kernel launch each;
    the expert of every row block selects the weight matrix), the activation is the usual
    fused elementwise kernel, and the outputs are gathered back and summed over the K choices
    with the routing weights in fp32.  Nothing synchronises with the host: ``R`` is the static
    bound ``pairs + E * (block - 1)`` rounded up to the block.

    With an ``expert`` mesh axis every rank keeps ``E / ep`` experts: tokens and routing decisions
    are all-gathered over the axis, each rank runs the pairs of its own experts, and a
    reduce-scatter sums the partial outputs back (the counterpart of the reference's ragged
    all-to-all pair, :2139-2178, with static sizes: per token the gather moves ``M`` values in
    and the scatter ``M`` values out per rank of the axis, independent of ``K``).
    """

    @config_class
    class Config(TransformerFeedForwardMoE.Config):
        seq_load_balance_loss_weight: Optional[float] = None
        # With experts sharded over the ``expert`` mesh axis: None sizes every rank's row buffer
        # for the worst case (all pairs of the axis choose this rank's experts; nothing is ever
        # dropped); a number caps it at that multiple of the fair share (``tokens * K`` rows),
        # and pairs beyond the cap are dropped as in the reference's approximate variant.
        expert_parallel_capacity: Optional[float] = None
        # Accepted for config compatibility with the reference (Pallas tile sizes / backend
        # choice); the grouped kernel has one tiling.
        tiling: Any = None
        gmm_backend: Any = None

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.gating = TopKDropFreeGating.default_config()
        cfg.num_groups = 1
        return cfg

    def _dispatch_and_combine(self, x: Tensor) -> Tensor:
        from axlearn_b200.ops import moe_ops

        cfg = self._config
        in_dtype = x.dtype
        token_shape = x.shape[:-1]
        m = cfg.input_dim
        x3 = x.reshape(x.shape[0], -1, m)                                        # [B, S, M]
        logits = torch.einsum("bsm,me->bse", x3.float(), self.parameters["gate_weight"].float())
        routing = self.gating(logits, cfg.seq_load_balance_loss_weight)
        aux = routing.load_balance_loss * cfg.load_balance_loss_weight
        if cfg.router_z_loss_weight:
            aux = aux + routing.router_z_loss * cfg.router_z_loss_weight
        if cfg.seq_load_balance_loss_weight and routing.seq_load_balance_loss is not None:
            aux = aux + routing.seq_load_balance_loss * cfg.seq_load_balance_loss_weight
        self.add_module_output("aux_loss", aux)

        k = routing.gate_assignment.shape[-1]
        tokens = x3.shape[0] * x3.shape[1]
        assignment = routing.gate_assignment.reshape(tokens, k)
        weights = routing.expert_weights.reshape(tokens, k)
        xt = x3.reshape(tokens, m)
        ep = self._expert_parallel_size()
        num_local, max_rows = cfg.num_experts, None
        if ep > 1:
            # Expert parallelism without a capacity: every rank of the expert axis sees the tokens
            # and routing decisions of the whole axis (all-gather), runs the pairs that chose ITS
            # experts through the grouped GEMMs, and the partial outputs are summed back to the
            # tokens' owners (reduce-scatter).  All sizes are static, so nothing waits for the
            # host; the blocks of the row buffer that stay unused are skipped by the kernels.
            num_local = cfg.num_experts // ep
            xt = coll.all_gather(xt, "expert", dim=0)
            weights = coll.all_gather(weights, "expert", dim=0)
            assignment = coll.all_gather_raw(assignment.contiguous(), current_mesh().group("expert"), ep, dim=0)
            local = assignment - coll.axis_index("expert") * num_local
            assignment = torch.where((local >= 0) & (local < num_local), local, torch.full_like(local, -1))
            if cfg.expert_parallel_capacity is not None:
                max_rows = int(math.ceil(cfg.expert_parallel_capacity * tokens * k))
        all_tokens = xt.shape[0]
        # Choice-major pair order decides the order inside an expert's run.
        dest_km, offsets, block_expert, rows = moe_ops.padded_group_layout(
            assignment.t().contiguous(), num_local, max_rows=max_rows)
        dest = dest_km.reshape(k, all_tokens).t().contiguous()                    # [T, K]
        xs = moe_ops.dispatch(xt, dest, rows)                                     # [R, M]
        ys = self._grouped_ffn(xs, offsets, block_expert)
        out = moe_ops.combine(ys, weights, dest)
        if ep > 1:
            out = coll.reduce_scatter(out, "expert", dim=0)
        return out.to(in_dtype).reshape(*token_shape, m)

    def _grouped_ffn(self, xs: Tensor, offsets: Tensor, block_expert: Tensor) -> Tensor:
        from axlearn_b200.ops import moe_ops

        cfg = self._config
        act = cfg.activation
        acts = list(act) if isinstance(act, tuple) else [act]
        names = [f"wi_{i}_weight" for i in range(len(acts))] if isinstance(act, tuple) else ["wi_weight"]
        wis = [self._expert_weight(n, "emh").to(xs.dtype) for n in names]
        wo = self._expert_weight("wo_weight", "ehm").to(xs.dtype)
        hs = [moe_ops.grouped_linear(xs, w, offsets, block_expert) for w in wis]
        if len(hs) == 2 and acts == ["nn.silu", "linear"]:
            h = ops.swiglu(hs[0], hs[1])
        else:
            h = None
            for hv, a in zip(hs, acts):
                hv = get_activation_fn(a)(hv)
                h = hv if h is None else h * hv
        h = self.dropout1(h) if "dropout1" in self._children else h
        return moe_ops.grouped_linear(h, wo, offsets, block_expert)


def convert_dense_to_moe_parameters(dense_params: dict, *, num_experts: int, activation: Union[str, tuple],
                                    gate_std: float = 0.02, generator: Optional[torch.Generator] = None) -> dict:
    """Parameters of a ``TransformerFeedForwardMoE`` initialised from a dense
    ``TransformerFeedForwardLayer`` ("sparse upcycling"; reference: :1843-2001): every expert
    starts as a copy of the dense FFN (``linear1[_i].weight -> wi[_i]_weight``,
    ``linear2.weight -> wo_weight``), the router is drawn at random, the norm is carried over."""
    out = {}
    names = [f"linear1_{i}" for i in range(len(activation))] if isinstance(activation, tuple) else ["linear1"]
    targets = [f"wi_{i}_weight" for i in range(len(activation))] if isinstance(activation, tuple) else ["wi_weight"]
    for src, dst in zip(names, targets):
        w = dense_params[src]["weight"]
        out[dst] = w.unsqueeze(0).repeat(num_experts, 1, 1).clone()
    w2 = dense_params["linear2"]["weight"]
    out["wo_weight"] = w2.unsqueeze(0).repeat(num_experts, 1, 1).clone()
    model_dim = w2.shape[1]
    out["gate_weight"] = torch.randn((model_dim, num_experts), generator=generator, dtype=w2.dtype) \
        .to(w2.device) * gate_std
    for key in ("norm", "prenorm", "postnorm"):
        if key in dense_params:
            out[key] = dense_params[key]
    return out


class ApproximateTokenDropFreeMoE(TransformerFeedForwardMoE):
    """Expert-parallel mixture of experts with drop-free *routing* and a generous fixed buffer
    (reference: axlearn/common/mixture_of_experts.py:2754-2824): the router picks top-k experts
    without any capacity limit, and every expert accepts up to ``expert_parallel_capacity`` times
    its fair share of assignments from each routing group, so tokens are only dropped under a
    load imbalance beyond that factor (reported as ``dropped_token_ratio``).  Everything after
    routing -- the exchange over peer memory or all-to-all, the expert GEMMs, the combine -- is
    the capacity-based machinery of the parent class with that buffer size."""

    @config_class
    class Config(TransformerFeedForwardMoE.Config):
        expert_parallel_capacity: float = 1.25
        seq_load_balance_loss_weight: Optional[float] = None

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.gating = TopKDropFreeGating.default_config()
        return cfg

    def _route(self, x: Tensor) -> tuple[Routing, Tensor]:
        """``x [O, G, S, M]`` -> routing with capacity slots, and the auxiliary loss."""
        cfg = self._config
        o, g, s, m = x.shape
        logits = torch.einsum("ogsm,me->ogse", x.float(), self.parameters["gate_weight"].float())
        free = self.gating(logits.reshape(o * g, s, cfg.num_experts), cfg.seq_load_balance_loss_weight)
        k = free.gate_assignment.shape[-1]
        index = free.gate_assignment.reshape(o, g, s, k)
        capacity = max(1, math.ceil(cfg.expert_parallel_capacity * s * k / cfg.num_experts))
        slot = _slots_in_priority_order(index, cfg.num_experts, capacity)
        kept = slot >= 0
        self.add_summary("dropped_token_ratio", 1.0 - kept.float().mean())
        weights = free.expert_weights.reshape(o, g, s, k) * kept.float()
        aux = free.load_balance_loss * cfg.load_balance_loss_weight
        if cfg.router_z_loss_weight:
            aux = aux + free.router_z_loss * cfg.router_z_loss_weight
        if cfg.seq_load_balance_loss_weight and free.seq_load_balance_loss is not None:
            aux = aux + free.seq_load_balance_loss * cfg.seq_load_balance_loss_weight
        routing = Routing(expert_index=index, slot=slot, weight=weights, num_experts=cfg.num_experts,
                          expert_capacity=capacity, load_balance_loss=free.load_balance_loss,
                          router_z_loss=free.router_z_loss)
        return routing, aux

    def _dispatch_and_combine(self, x: Tensor) -> Tensor:
        cfg = self._config
        in_dtype = x.dtype
        token_shape = x.shape[:-1]
        o = cfg.outer_batch
        tokens = math.prod(token_shape) // o
        if tokens % cfg.num_groups:
            raise ValueError(f"{tokens} tokens per outer batch must be divisible by num_groups({cfg.num_groups}).")
        x = x.reshape(o, cfg.num_groups, tokens // cfg.num_groups, cfg.input_dim)
        routing, aux = self._route(x)
        self.add_module_output("aux_loss", aux)
        fused = self._peer_exchange(x, routing)
        if fused is not None:
            return fused.to(in_dtype).reshape(*token_shape, cfg.input_dim)
        expert_in = self.gating.dispatch(x, routing)
        expert_out = self._experts(expert_in)
        out = self.gating.combine(expert_out, routing, dtype=in_dtype)
        return out.reshape(*token_shape, cfg.input_dim)
