"""Module / invocation-context / BaseLayer behaviour (mirrors the cases of the reference's
axlearn/common/module_test.py and base_layer_test.py that the layer library relies on)."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec, RematSpec, nothing_saveable
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.module import Module, current_context, functional, nowrap
from axlearn_b200.common.param_init import constant_initializer
from axlearn_b200.common.utils import flatten_items


class Affine(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED

    def _create_layer_parameter_specs(self):
        d = self._config.dim
        return {"weight": ParameterSpec(shape=(d, d)),
                "bias": ParameterSpec(shape=(d,), initializer=constant_initializer(0.5))}

    def forward(self, x):
        y = x @ self.parameters["weight"] + self.parameters["bias"]
        self.add_summary("mean", y.mean().detach())
        self.add_module_output("y", y)
        return y

    @nowrap
    def helper(self):
        return "no context needed"


class Stack(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED
        n: int = 2
        layer: InstantiableConfig = Affine.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        for i in range(cfg.n):
            self._add_child(f"l{i}", cfg.layer.clone(dim=cfg.dim))

    def forward(self, x):
        for i in range(self._config.n):
            x = getattr(self, f"l{i}")(x)
        self.add_state_update("calls", torch.tensor(1))
        return x

    def uses_key(self):
        return self.prng_key, self.l0.uses_parent_key()


def _stack(n=2):
    return Stack.default_config().set(name="root", dim=4, n=n).instantiate(parent=None)


def test_children_paths_and_specs():
    m = _stack()
    assert list(m.children) == ["l0", "l1"] and m.l1.path() == "root.l1" and m.l1.parent is m
    specs = m.create_parameter_specs_recursively()
    assert [p for p, _ in flatten_items(specs)] == ["l0/bias", "l0/weight", "l1/bias", "l1/weight"]
    assert specs["l0"]["weight"].shape == (4, 4)
    with pytest.raises(Exception):
        m._add_child("l0", Affine.default_config().set(dim=4))  # pylint: disable=protected-access


def test_initialisation_is_deterministic_and_per_child():
    m = _stack()
    p1 = m.initialize_parameters_recursively(prng.PRNGKey(0))
    p2 = m.initialize_parameters_recursively(prng.PRNGKey(0))
    p3 = m.initialize_parameters_recursively(prng.PRNGKey(1))
    assert torch.equal(p1["l0"]["weight"], p2["l0"]["weight"]) and not torch.equal(p1["l0"]["weight"], p3["l0"]["weight"])
    assert not torch.equal(p1["l0"]["weight"], p1["l1"]["weight"])      # children get different keys
    assert torch.equal(p1["l0"]["bias"], torch.full((4,), 0.5))
    # Prebuilt leaves are kept as given.
    pre = {"l0": {"weight": torch.zeros(4, 4)}}
    p4 = m.initialize_parameters_recursively(prng.PRNGKey(0), prebuilt=pre)
    assert torch.equal(p4["l0"]["weight"], torch.zeros(4, 4)) and torch.equal(p4["l1"]["weight"], p1["l1"]["weight"])


def test_functional_collects_outputs_per_path():
    m = _stack()
    params = m.initialize_parameters_recursively(prng.PRNGKey(0))
    x = torch.randn(3, 4)
    y, oc = functional(m, prng.PRNGKey(1), params, [x], is_training=True, drop_output_collections=())
    ref = (x @ params["l0"]["weight"] + 0.5) @ params["l1"]["weight"] + 0.5
    assert torch.allclose(y, ref)
    assert set(oc.summaries) == {"l0", "l1"} and "mean" in oc.summaries["l0"]
    assert torch.allclose(oc.module_outputs["l1"]["y"], ref)
    assert oc.state_updates["calls"] == 1
    # module_outputs are dropped by default.
    _, oc2 = functional(m, prng.PRNGKey(1), params, [x], is_training=True)
    assert not flatten_items(oc2.module_outputs)
    assert current_context() is None


def test_methods_need_a_context_unless_nowrap():
    m = _stack()
    with pytest.raises(RuntimeError, match="invocation context"):
        m.forward(torch.zeros(1, 4))
    assert m.l0.helper() == "no context needed"


def test_state_is_scoped_to_the_child():
    class Peek(Affine):
        def forward(self, x):
            assert set(self.state) == {"weight", "bias"}          # only this layer's own parameters
            assert self.is_training is False
            return super().forward(x)

    m = Stack.default_config().set(name="root", dim=4, n=1, layer=Peek.default_config()).instantiate(parent=None)
    params = m.initialize_parameters_recursively(prng.PRNGKey(0))
    functional(m, None, params, [torch.zeros(1, 4)], is_training=False)


def test_prng_keys_fold_in_child_names():
    class Keyed(Affine):
        def uses_parent_key(self):
            return self.prng_key

    m = Stack.default_config().set(name="root", dim=4, n=2, layer=Keyed.default_config()).instantiate(parent=None)
    params = m.initialize_parameters_recursively(prng.PRNGKey(0))
    (root_key, child_key), _ = functional(m, prng.PRNGKey(7), params, [], is_training=True, method="uses_key")
    assert torch.equal(root_key, prng.PRNGKey(7)) and not torch.equal(child_key, root_key)
    (_, again), _ = functional(m, prng.PRNGKey(7), params, [], is_training=True, method="uses_key")
    assert torch.equal(child_key, again)
    # Without a key, asking for one is an error rather than silent determinism.
    with pytest.raises(Exception):
        functional(m, None, params, [], is_training=True, method="uses_key")


def test_remat_spec_recomputes_and_matches_gradients():
    calls = {"n": 0}

    class Counting(Affine):
        def forward(self, x):
            calls["n"] += 1
            return torch.tanh(super().forward(x))

    def build(remat):
        child = Counting.default_config()
        if remat:
            child.remat_spec = RematSpec(prevent_cse=False, policy=nothing_saveable)
        return Stack.default_config().set(name="root", dim=4, n=1, layer=child).instantiate(parent=None)

    x = torch.randn(5, 4)
    grads = []
    for remat in (False, True):
        calls["n"] = 0
        layer = build(remat)
        params = layer.initialize_parameters_recursively(prng.PRNGKey(0))
        params = {"l0": {k: v.clone().requires_grad_(True) for k, v in params["l0"].items()}}
        y, _ = functional(layer, None, params, [x], is_training=True)
        y.square().sum().backward()
        grads.append(params["l0"]["weight"].grad.clone())
        assert calls["n"] == (2 if remat else 1)      # replayed once in backward
    assert torch.allclose(grads[0], grads[1], atol=1e-6)


def test_parameter_dtype_and_weight_decay_scale_in_specs():
    class Typed(BaseLayer):
        def _create_layer_parameter_specs(self):
            return {"scale": ParameterSpec(shape=(2,), dtype=torch.float64, weight_decay_scale=0.0)}

    layer = Typed.default_config().set(name="t").instantiate(parent=None)
    spec = layer.create_parameter_specs_recursively()["scale"]
    assert spec.dtype == torch.float64 and spec.weight_decay_scale == 0.0
    assert layer.initialize_parameters_recursively(prng.PRNGKey(0))["scale"].dtype == torch.float64
