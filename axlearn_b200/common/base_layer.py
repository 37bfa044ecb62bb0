"""BaseLayer: declarative parameters, sharding specs, rematerialisation, tensor stats.

A layer lists its parameters as ``ParameterSpec``s (global shape, dtype, mesh axes,
initialiser, fan axes, weight-decay scale).  ``initialize_parameters_recursively`` turns the
spec tree into a nested dict of tensors holding *this rank's shard*: the mesh in scope
decides the local shape, and the values are the corresponding slice of the globally-defined
random tensor, so a model initialised on 1 GPU and on 8 GPUs holds identical numbers.

Rematerialisation is a wrapper around any public method: with ``remat_spec`` set and
training on, the method runs without recording autograd state, keeps only its tensor inputs
and the layer's parameters, and is replayed under autograd when gradients arrive.  There is
no tracing compiler, so the save policy is binary: ``everything_saveable`` disables remat,
any other policy (``nothing_saveable`` being the canonical one) keeps nothing but inputs.
Fused kernels that can cheaply keep extra residuals (flash-attention output + LSE) do so
themselves.

Parity targets in the reference (axlearn/common/base_layer.py): ``ParameterSpec`` (:165-227),
``RematSpec`` (:235), ``TensorStats`` (:271-415), remat of wrapped methods (:520-596),
dtype / param_init inheritance (:598-610), ``_create_layer_parameter_specs`` (:613),
``create_parameter_specs_recursively`` (:617), ``initialize_parameters_recursively``
(:651-703), default fan axes (:773-781), ``_remat_name`` (:783-797), ``no_remat`` (:871).
"""

from __future__ import annotations

import dataclasses
import math
from typing import Any, Callable, Optional, Sequence, Union

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.config import (
    REQUIRED,
    Configurable,
    ConfigOr,
    InstantiableConfig,
    Required,
    config_class,
    maybe_instantiate,
)
from axlearn_b200.common.module import (
    Module,
    current_context,
    new_output_collection,
    nowrap,
    set_current_context,
)
from axlearn_b200.common.param_init import DefaultInitializer, FanAxes, Initializer
from axlearn_b200.common.utils import (
    Nested,
    NestedTensor,
    PartitionSpec,
    TensorSpec,
    flatten_items,
    tree_map,
)
from axlearn_b200.parallel.mesh import current_mesh

Tensor = torch.Tensor


@dataclasses.dataclass
class FactorizationSpec:
    """Which axes Adafactor-style optimisers may factorise: one entry per dim, each None,
    "row" or "col"."""

    axes: Sequence[Optional[str]]

    __config_value__ = True


@dataclasses.dataclass
class ParameterSpec(TensorSpec):
    """Everything needed to create, shard and regularise one parameter."""

    initializer: Optional[Any] = None  # Initializer instance or config.
    factorization: Optional[FactorizationSpec] = None
    fan_axes: Optional[FanAxes] = None
    weight_decay_scale: Optional[float] = None
    memory_kind: Optional[str] = None  # "device" (default) or "pinned_host".

    def fans(self) -> dict[str, float]:
        from axlearn_b200.common.param_init import compute_fans

        if self.fan_axes is None:
            raise ValueError("fan_axes is not set")
        fan_in, fan_out = compute_fans(self.shape, self.fan_axes)
        return {"fan_in": fan_in, "fan_out": fan_out, "fan_avg": (fan_in + fan_out) / 2}


NestedParameterSpec = Union[ParameterSpec, dict]


# Remat policies.  ``everything_saveable`` switches rematerialisation off, ``nothing_saveable``
# keeps only a layer's inputs; the selective policies (by tagged name, all projection GEMMs, with
# or without offload to pinned host memory) live in ``axlearn_b200.common.remat``.
def everything_saveable(*_, **__):
    return True


def nothing_saveable(*_, **__):
    return False


from axlearn_b200.common.remat import (  # noqa: E402  pylint: disable=wrong-import-position
    dots_saveable,
    offload_dots_saveable,
    save_and_offload_only_these_names_regex,
    save_only_these_names,
    save_only_these_names_regex,
)


@dataclasses.dataclass
class RematSpec:
    """Rematerialisation request for a layer's wrapped methods."""

    prevent_cse: bool = True
    policy: Optional[Any] = None  # Callable or config thereof; None == nothing_saveable.

    __config_value__ = True

    def saves_everything(self) -> bool:
        pol = maybe_instantiate(self.policy) if isinstance(self.policy, InstantiableConfig) else self.policy
        return pol is everything_saveable

    def selective_policy(self):
        """The ``remat.RematPolicy`` that names what a replayed layer keeps, or None (keep inputs
        only)."""
        from axlearn_b200.common import remat

        return remat.as_policy(self.policy)


@dataclasses.dataclass
class TensorRMSNorm:
    """Expected range of the RMS of a tensor; summaries flag values outside it."""

    min_value: Optional[float] = None
    max_value: Optional[float] = None


class TensorStats(Module):
    """Computes statistics of a tensor and reports them as summaries."""

    @config_class
    class Config(Module.Config):
        inline_child_summaries: bool = False

    def add_stats(self, name: str, value: Tensor) -> None:
        raise NotImplementedError(type(self))


class CompositeTensorStats(TensorStats):
    @config_class
    class Config(TensorStats.Config):
        tensor_stats: dict[str, InstantiableConfig] = {}

    def __init__(self, cfg, *, parent):
        super().__init__(cfg, parent=parent)
        self._kids = [self._add_child(n, c) for n, c in cfg.tensor_stats.items()]

    def add_stats(self, name: str, value: Tensor) -> None:
        for k in self._kids:
            k.add_stats(name, value)


class TensorRMSNormStats(TensorStats):
    def add_stats(self, name: str, value: Tensor) -> None:
        v = value.detach().float()
        self.add_summary(f"{name}_rms_norm", v.pow(2).mean().sqrt())


class TensorMaxAbsStats(TensorStats):
    def add_stats(self, name: str, value: Tensor) -> None:
        self.add_summary(f"{name}_max_abs", value.detach().abs().max())


class DefaultTensorStats(CompositeTensorStats):
    @config_class
    class Config(CompositeTensorStats.Config):
        tensor_stats: dict[str, InstantiableConfig] = {
            "norm": TensorRMSNormStats.default_config(),
            "max_abs": TensorMaxAbsStats.default_config(),
        }


class ParameterNoise(Configurable):
    """Interface for perturbing a layer's parameters during training (reference:
    axlearn/common/base_layer.py:263-269).  ``apply`` returns a tree of the same structure;
    it must not modify ``params`` in place."""

    def apply(self, prng_key: Tensor, params: Any) -> Any:
        raise NotImplementedError(type(self))


class GaussianParameterNoise(ParameterNoise):
    """Adds ``std * N(0, 1)`` to every floating-point parameter whose name matches ``regex``."""

    @config_class
    class Config(Configurable.Config):
        std: float = 0.0
        regex: str = ".*"

    def apply(self, prng_key: Tensor, params: Any) -> Any:
        import re

        cfg = self._config
        items = flatten_items(params)
        keys = prng.split(prng_key, max(1, len(items)))
        out = []
        for (path, value), key in zip(items, keys):
            if isinstance(value, Tensor) and value.is_floating_point() and re.fullmatch(cfg.regex, path):
                noise = prng.normal(key, value.shape, dtype=value.dtype, device=value.device, std=cfg.std)
                value = value + noise  # differentiable: the gradient reaches the clean parameter
            out.append((path, value))
        from axlearn_b200.common.utils import unflatten_items

        return unflatten_items(out) if out else params


# --------------------------------------------------------------------------------------
# Remat machinery.
# --------------------------------------------------------------------------------------

_remat_disabled_depth = 0


class _Remat(torch.autograd.Function):
    """Runs ``run(tensors) -> tuple[Tensor]`` keeping only ``tensors`` for backward."""

    @staticmethod
    def forward(ctx, run, policy, *tensors):  # pylint: disable=arguments-differ
        from axlearn_b200.common import remat
        from axlearn_b200.parallel.mesh import current_mesh

        ctx.stash = remat.LayerStash(policy) if policy is not None else None

        ctx.run = run
        ctx.needs = [t.requires_grad for t in tensors]
        # The replay runs on an autograd worker thread, whose thread-local mesh stack is empty.
        ctx.mesh = current_mesh()
        ctx.save_for_backward(*tensors)
        with torch.no_grad(), remat.recording(ctx.stash):
            outs = run(tensors, first_pass=True)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):  # pylint: disable=arguments-differ
        from axlearn_b200.parallel.mesh import current_mesh

        if ctx.mesh is not None and current_mesh() is not ctx.mesh:
            with ctx.mesh:
                return _Remat._backward(ctx, *grads)
        return _Remat._backward(ctx, *grads)

    @staticmethod
    def _backward(ctx, *grads):
        tensors = ctx.saved_tensors
        replay = [
            t.detach().requires_grad_(need) if t.is_floating_point() else t.detach()
            for t, need in zip(tensors, ctx.needs)
        ]
        from axlearn_b200.common import remat

        with torch.enable_grad(), remat.replaying(ctx.stash):
            outs = ctx.run(replay, first_pass=False)
        if ctx.stash is not None:
            ctx.stash.clear()
        pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(
            (r.grad if need and r.is_floating_point() else None)
            for r, need in zip(replay, ctx.needs)
        )


def _flatten_tensors(tree: Any) -> tuple[list[Tensor], Callable[[Sequence[Tensor]], Any]]:
    """Splits a tree into its tensor leaves and a function that rebuilds the tree from a
    replacement list of tensors (non-tensor leaves are kept)."""
    tensors: list[Tensor] = []

    def strip(x):
        if isinstance(x, torch.Tensor):
            tensors.append(x)
            return _Slot(len(tensors) - 1)
        return x

    skeleton = tree_map(strip, tree, is_leaf=lambda x: isinstance(x, torch.Tensor))

    def rebuild(new: Sequence[Tensor]):
        return tree_map(
            lambda x: new[x.i] if isinstance(x, _Slot) else x,
            skeleton,
            is_leaf=lambda x: isinstance(x, _Slot),
        )

    return tensors, rebuild


@dataclasses.dataclass(frozen=True)
class _Slot:
    i: int


def remat_call(fn: Callable, *, state: Any, args: tuple, kwargs: dict, policy: Any = None) -> Any:
    """Calls ``fn(*args, **kwargs)`` in the current invocation context with
    rematerialisation: only the tensor leaves of (state, args, kwargs) are kept, plus what the
    selective ``policy`` (a ``remat.RematPolicy``) names."""
    ctx = current_context()
    in_tensors, rebuild_inputs = _flatten_tensors({"state": state, "args": args, "kwargs": kwargs})
    out_box: dict[str, Any] = {}

    def run(tensors, *, first_pass: bool):
        tree = rebuild_inputs(list(tensors))
        # First pass writes summaries into the live collection; the replay's are discarded.
        oc = ctx.output_collection if first_pass else new_output_collection()
        replay_ctx = dataclasses.replace(ctx, state=tree["state"], output_collection=oc)
        with set_current_context(replay_ctx, require_parent=False):
            out = fn(*tree["args"], **tree["kwargs"])
        out_tensors, rebuild_out = _flatten_tensors(out)
        if first_pass:
            out_box["rebuild"] = rebuild_out
        return out_tensors

    outs = _Remat.apply(run, policy, *in_tensors)
    return out_box["rebuild"](list(outs))


class no_remat:  # pylint: disable=invalid-name
    """Context manager / decorator disabling remat for the calls it encloses."""

    def __init__(self, fn: Optional[Callable] = None):
        self._fn = fn

    def __enter__(self):
        global _remat_disabled_depth
        _remat_disabled_depth += 1

    def __exit__(self, *exc):
        global _remat_disabled_depth
        _remat_disabled_depth -= 1

    def __call__(self, *args, **kwargs):
        with self:
            return self._fn(*args, **kwargs)


# --------------------------------------------------------------------------------------
# BaseLayer.
# --------------------------------------------------------------------------------------


class BaseLayer(Module):
    """A Module with parameters."""

    @config_class
    class Config(Module.Config):
        # Parameter dtype; inherited from the parent when None.
        dtype: Optional[torch.dtype] = None
        # Initialiser config; inherited from the parent when None.
        param_init: Optional[InstantiableConfig] = None
        # Mesh axes of this layer's parameters (per-dim); layer-specific defaults apply.
        param_partition_spec: Optional[Sequence[Any]] = None
        remat_spec: Optional[RematSpec] = None
        # Parameter perturbation, applied by the trainer through
        # apply_parameter_noise_recursively() (never implicitly inside forward).
        param_noise: Optional[InstantiableConfig] = None
        tensor_stats: Optional[InstantiableConfig] = None

    def __init__(self, cfg: "BaseLayer.Config", *, parent: Optional[Module] = None):
        super().__init__(cfg, parent=parent)
        self._param_noise = cfg.param_noise.instantiate() if cfg.param_noise is not None else None
        self._param_init: Optional[Initializer] = (
            cfg.param_init.instantiate() if cfg.param_init is not None else None
        )
        if cfg.tensor_stats is not None:
            self._add_child("tensor_stats", cfg.tensor_stats)

    # ------------------------------------------------------------------ inheritance
    @nowrap
    def dtype(self) -> torch.dtype:
        if self._config.dtype is not None:
            return self._config.dtype
        if isinstance(self._parent, BaseLayer):
            return self._parent.dtype()
        return torch.float32

    @nowrap
    def param_init(self) -> Initializer:
        if self._param_init is not None:
            return self._param_init
        if isinstance(self._parent, BaseLayer):
            return self._parent.param_init()
        self._param_init = DefaultInitializer.default_config().instantiate()
        return self._param_init

    # ------------------------------------------------------------------ remat hook
    def _call_in_context(self, fn: Callable, args: tuple, kwargs: dict) -> Any:
        spec = self._config.remat_spec
        ctx = current_context()
        if (
            spec is not None
            and not spec.saves_everything()
            and _remat_disabled_depth == 0
            and ctx is not None
            and ctx.is_training
            and torch.is_grad_enabled()
            and not getattr(fn, "__no_remat__", False)
        ):
            bound = lambda *a, **k: fn(self, *a, **k)
            return remat_call(bound, state=ctx.state, args=args, kwargs=kwargs, policy=spec.selective_policy())
        return fn(self, *args, **kwargs)

    # ------------------------------------------------------------------ parameter noise
    @nowrap
    def has_parameter_noise(self) -> bool:
        if self._param_noise is not None:
            return True
        return any(isinstance(c, BaseLayer) and c.has_parameter_noise() for c in self._children.values())

    @nowrap
    def apply_parameter_noise_recursively(self, prng_key: Tensor, params: Any) -> Any:
        """Returns ``params`` with every configured ``param_noise`` applied: children first (one
        key split per BaseLayer child, in declaration order), then this layer's own noise on the
        result.  The input tree is not modified (reference: axlearn/common/base_layer.py:747-771)."""
        if not self.has_parameter_noise():
            return params
        params = type(params)(**params) if isinstance(params, dict) else params
        for name, child in self._children.items():
            if not isinstance(child, BaseLayer):
                continue
            prng_key, child_key = prng.split(prng_key, 2)
            if isinstance(params, dict) and name in params:
                params[name] = child.apply_parameter_noise_recursively(child_key, params[name])
        if self._param_noise is not None:
            params = self._param_noise.apply(prng_key, params)
        return params

    # ------------------------------------------------------------------ parameter specs
    def _create_layer_parameter_specs(self) -> dict[str, ParameterSpec]:
        """Specs of the parameters owned directly by this layer (not its children)."""
        return {}

    @nowrap
    def create_parameter_specs_recursively(self) -> NestedParameterSpec:
        specs: dict[str, Any] = {}
        for name, spec in self._create_layer_parameter_specs().items():
            spec = dataclasses.replace(spec)
            if spec.dtype is None:
                spec.dtype = self.dtype()
            if spec.initializer is None:
                spec.initializer = self.param_init()
            if spec.fan_axes is None:
                spec.fan_axes = self._compute_fan_axes(name, spec)
            specs[name] = spec
        for name, child in self._children.items():
            if not isinstance(child, BaseLayer):
                continue
            if name in specs:
                raise ValueError(f"{self.path()}: child {name} collides with a parameter")
            child_specs = child.create_parameter_specs_recursively()
            if child_specs != {} or True:
                specs[name] = child_specs
        return specs

    def _compute_fan_axes(self, name: str, parameter_spec: ParameterSpec) -> Optional[FanAxes]:
        """Default: 2-D ``*weight`` uses in=-2, out=-1; others have no fans."""
        if not name.endswith("weight"):
            return None
        if len(parameter_spec.shape) != 2:
            raise NotImplementedError(
                f"{type(self).__name__}: fan axes must be given for {name} with shape "
                f"{tuple(parameter_spec.shape)}"
            )
        return FanAxes(in_axis=-2, out_axis=-1)

    # ------------------------------------------------------------------ initialisation
    @nowrap
    def initialize_parameters_recursively(
        self,
        prng_key: torch.Tensor,
        *,
        prebuilt: Optional[Nested] = None,
        device: Union[str, torch.device, None] = None,
    ) -> NestedTensor:
        """Returns ``{name: tensor | subtree}`` for this layer and its children.

        The key is split once per own parameter, then once per child, in declaration order;
        a split is consumed even when the value comes from ``prebuilt`` so that the other
        parameters do not depend on which ones were prebuilt.
        """
        if device is None:
            device = default_device()
        own = self._create_layer_parameter_specs()
        kids = [(n, c) for n, c in self._children.items() if isinstance(c, BaseLayer)]
        keys = prng.split(prng_key, len(own) + len(kids)) if (own or kids) else []
        params: dict[str, Any] = {}
        specs = self.create_parameter_specs_recursively()
        for i, name in enumerate(own):
            pre = prebuilt.get(name) if isinstance(prebuilt, dict) else None
            if isinstance(pre, torch.Tensor):
                params[name] = pre
            else:
                params[name] = self._initialize_parameter(
                    name, prng_key=keys[i], parameter_spec=specs[name], device=device
                )
        for j, (name, child) in enumerate(kids):
            pre = prebuilt.get(name) if isinstance(prebuilt, dict) else None
            params[name] = child.initialize_parameters_recursively(
                keys[len(own) + j], prebuilt=pre, device=device
            )
        return params

    def _initialize_parameter(
        self, name: str, *, prng_key: torch.Tensor, parameter_spec: ParameterSpec, device
    ) -> Tensor:
        """Creates this rank's shard of one parameter."""
        init = parameter_spec.initializer
        if isinstance(init, InstantiableConfig):
            init = init.instantiate()
        full = init.initialize(
            name,
            prng_key=prng_key,
            shape=tuple(parameter_spec.shape),
            dtype=parameter_spec.dtype,
            axes=parameter_spec.fan_axes,
            device=device,
        )
        return shard_tensor(full, parameter_spec.mesh_axes)

    # ------------------------------------------------------------------ runtime helpers
    @property
    def parameters(self) -> NestedTensor:
        return self.state

    def _remat_name(self, x: Tensor, name: str) -> Tensor:
        """Tags ``x`` as ``"{ClassName}.{name}"`` for save policies.  The eager runtime has
        no selective policy, so the tag is informational (it names an NVTX marker)."""
        return x

    def _add_tensor_stats(self, name: str, value: Tensor) -> None:
        if "tensor_stats" in self._children:
            self._children["tensor_stats"].add_stats(name, value)

    def _add_activation_summary(
        self, *, name: str, activations: Tensor, activation_paddings: Optional[Tensor] = None
    ) -> None:
        a = activations.detach().float()
        if activation_paddings is None:
            mean = a.mean()
            norm = a.pow(2).sum(-1).sqrt().mean()
        else:
            w = (1 - activation_paddings.float()).unsqueeze(-1)
            denom = w.sum().clamp_min(1.0)
            mean = (a * w).sum() / (denom * a.shape[-1])
            norm = (a.pow(2).sum(-1, keepdim=True).sqrt() * w).sum() / denom
        self.add_summary(f"activations/{name}_mean", mean)
        self.add_summary(f"activations/{name}_norm", norm)


# --------------------------------------------------------------------------------------
# Sharding helpers.
# --------------------------------------------------------------------------------------

_default_device: list = [None]


def default_device() -> torch.device:
    if _default_device[0] is not None:
        return _default_device[0]
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


class use_device:  # pylint: disable=invalid-name
    """Scopes the device on which parameters are created."""

    def __init__(self, device):
        self._device = torch.device(device)

    def __enter__(self):
        self._prev = _default_device[0]
        _default_device[0] = self._device

    def __exit__(self, *exc):
        _default_device[0] = self._prev


def shard_tensor(full: Tensor, mesh_axes: Optional[Sequence[Any]]) -> Tensor:
    """This rank's shard of ``full`` under the mesh in scope (a contiguous copy)."""
    mesh = current_mesh()
    if mesh is None or mesh_axes is None or mesh.size == 1:
        return full
    slices = mesh.shard_slices(full.shape, mesh_axes)
    if all(s.start == 0 and s.stop == d for s, d in zip(slices, full.shape)):
        return full
    return full[slices].contiguous()


def local_shape(spec: TensorSpec) -> tuple[int, ...]:
    mesh = current_mesh()
    if mesh is None or spec.mesh_axes is None:
        return tuple(spec.shape)
    return mesh.shard_shape(spec.shape, spec.mesh_axes)


def param_count(specs: NestedParameterSpec) -> int:
    return sum(math.prod(s.shape) for _, s in flatten_items(specs, is_leaf=lambda x: isinstance(x, TensorSpec)))
