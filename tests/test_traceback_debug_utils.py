"""Module-path notes on exceptions and the non-finite output checks."""

import traceback

import pytest
import torch

from axlearn_b200.common import debug_utils, traceback_util
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import config_class
from axlearn_b200.common.module import functional


class Leaf(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        mode: str = "ok"

    def forward(self, x):
        mode = self._config.mode
        if mode == "raise":
            raise ValueError("boom")
        if mode == "nan":
            return x / torch.zeros_like(x) * 0.0
        if mode == "inf":
            return {"y": (x.abs() + 1) / torch.zeros_like(x)}
        return x + 1


class Tower(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        bad: str = "ok"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("good", Leaf.default_config())
        self._add_child("bad", Leaf.default_config().set(mode=cfg.bad))

    def forward(self, x):
        return self.bad(self.good(x))


def _run(bad):
    layer = Tower.default_config().set(name="tower", bad=bad).instantiate(parent=None)
    return functional(layer, None, {"good": {}, "bad": {}}, [torch.ones(3)], is_training=False)


def test_exception_carries_the_module_stack():
    with pytest.raises(ValueError, match="boom") as info:
        _run("raise")
    assert traceback_util.module_stack(info.value) == ["tower.bad"]         # the root call is the caller itself
    text = "".join(traceback.format_exception(info.value))
    assert "in module tower.bad [Leaf.forward]" in text
    traceback_util.set_stack_summary_enabled(False)
    try:
        with pytest.raises(ValueError) as info2:
            _run("raise")
        assert traceback_util.module_stack(info2.value) == []
    finally:
        traceback_util.set_stack_summary_enabled(None)


def test_annotate_and_no_summary():
    @traceback_util.annotate_stack(stage="restore", step=7)
    def outer():
        raise KeyError("k")

    with pytest.raises(KeyError) as info:
        outer()
    assert traceback_util.annotations(info.value) == [{"stage": "restore", "step": "7"}]

    @traceback_util.annotate_stack(stage="iter")
    @traceback_util.no_stack_summary
    def quiet():
        raise StopIteration

    with pytest.raises(StopIteration) as info:
        quiet()
    assert traceback_util.annotations(info.value) == []
    wrapped = traceback_util.wrap(outer, path=lambda: "a.b", cls="C")
    with pytest.raises(KeyError) as info:
        wrapped()
    assert traceback_util.module_stack(info.value) == ["a.b"]


def test_first_module_with_a_non_finite_output_is_named():
    out, _ = _run("nan")                                          # no checks: NaNs pass silently
    assert torch.isnan(out).all()
    with debug_utils.check_module_outputs():
        with pytest.raises(FloatingPointError, match=r"NaN in an output of tower\.bad \[Leaf\.forward\]"):
            _run("nan")
        with pytest.raises(FloatingPointError, match=r"infinity in an output of tower\.bad"):
            _run("inf")
        out, _ = _run("ok")
        assert torch.equal(out, torch.full((3,), 3.0))
    with debug_utils.check_module_outputs(errors=[debug_utils.NAN]):
        assert torch.isinf(_run("inf")[0]["y"]).all()            # only NaNs are checked here
    assert debug_utils.active_checks() is None


def test_guard_index():
    idx = torch.tensor([0, 3, 2])
    assert debug_utils.guard_index(idx, 4) is idx
    with pytest.raises(IndexError, match=r"token ids: values span \[0, 3\]"):
        debug_utils.guard_index(idx, 3, what="token ids")
    with pytest.raises(IndexError):
        debug_utils.guard_index(torch.tensor([-1]), 3)
