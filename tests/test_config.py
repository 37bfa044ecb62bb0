"""Config system behaviour (mirrors the cases of the reference's axlearn/common/config_test.py
that downstream code relies on)."""

import copy
import dataclasses
import pickle
from typing import Optional

import pytest

from axlearn_b200.common import config
from axlearn_b200.common.config import (
    REQUIRED,
    Configurable,
    InstantiableConfig,
    Required,
    config_class,
    config_for_class,
    config_for_function,
    maybe_set_config,
)


@config_class
class Point(config.ConfigBase):
    x: Required[int] = REQUIRED
    y: int = 2
    tags: list = []
    inner: Optional[config.ConfigBase] = None


class Layer(Configurable):
    @config_class
    class Config(Configurable.Config):
        dim: Required[int] = REQUIRED
        scale: float = 1.0
        child: Optional[InstantiableConfig] = None

    def __init__(self, cfg):
        super().__init__(cfg)
        self.child = cfg.child.instantiate() if cfg.child is not None else None


def test_fields_defaults_and_set_chaining():
    p = Point()
    assert p.y == 2 and p.x is REQUIRED and not p.x
    assert p.set(x=1, y=3) is p and (p.x, p.y) == (1, 3)
    assert "x" in p and "z" not in p and p.keys() == ["x", "y", "tags", "inner"]
    assert len(p) == 4 and dict(p.items())["y"] == 3


def test_unknown_field_suggests_similar_names():
    p = Point()
    with pytest.raises(config.UnknownFieldError) as e:
        p.set(tag=[1])
    assert "tags" in str(e.value)
    with pytest.raises(config.UnknownFieldError):
        _ = p.does_not_exist
    with pytest.raises(AttributeError):
        del p.x


def test_mutable_values_are_copied_on_set_and_default():
    tags = [1, 2]
    a, b = Point(), Point()
    a.set(tags=tags)
    tags.append(3)
    assert a.tags == [1, 2]          # by value
    a.tags.append(9)
    assert b.tags == []              # defaults are not shared between instances
    inner = Point().set(x=5)
    a.inner = inner
    inner.x = 6
    assert a.inner.x == 5


def test_field_name_and_value_validation():
    with pytest.raises(config.InvalidConfigNameError):
        config.validate_config_field_name("BadName")
    with pytest.raises(config.InvalidConfigNameError):
        config.validate_config_field_name("_private")
    config.validate_config_field_name("ok_name_2")

    class Opaque:
        pass

    with pytest.raises(config.InvalidConfigValueError):
        Point().set(y=Opaque())
    Point().set(tags=[(1, "a"), {"k": 2.0}])   # nested plain containers are fine

    with pytest.raises(config.NonConfigFieldError):
        @config_class
        class Bad(config.ConfigBase):  # pylint: disable=unused-variable
            x: int = 1
            forgot_the_annotation = 3


def test_required_fields_checked_at_instantiate():
    with pytest.raises(config.RequiredFieldMissingError) as e:
        Layer.default_config().instantiate()
    assert "dim" in str(e.value)
    nested = Layer.default_config().set(dim=4, child=Layer.default_config())
    with pytest.raises(config.RequiredFieldMissingError) as e:
        nested.instantiate()
    assert "child" in str(e.value) and "dim" in str(e.value)
    nested.child.dim = 2
    layer = nested.instantiate()
    assert isinstance(layer.child, Layer) and layer.child.config.dim == 2


def test_instance_config_is_a_private_copy():
    cfg = Layer.default_config().set(dim=4)
    layer = cfg.instantiate()
    cfg.dim = 8
    assert layer.config.dim == 4
    layer.config.dim = 16            # mutating the returned copy does not affect the instance
    assert layer.config.dim == 4


def test_clone_equality_copy_pickle():
    a = Layer.default_config().set(dim=4, child=Layer.default_config().set(dim=1))
    b = a.clone(scale=2.0)
    assert a.scale == 1.0 and b.scale == 2.0 and b.child == a.child and b.child is not a.child
    assert a != b and a == a.clone() and a == copy.deepcopy(a)
    assert pickle.loads(pickle.dumps(a)) == a
    assert REQUIRED is copy.deepcopy(REQUIRED) and pickle.loads(pickle.dumps(REQUIRED)) is REQUIRED


def test_get_set_recursively_and_flat_dict():
    a = Layer.default_config().set(dim=4, child=Layer.default_config().set(dim=1))
    assert a.get_recursively(["child", "dim"]) == 1
    a.set_recursively(["child", "scale"], value=3.0)
    assert a.child.scale == 3.0
    with pytest.raises(AttributeError):
        a.set_recursively(["child", "nope"], value=1)
    flat = a.to_flat_dict(omit_default_values={})
    assert flat["dim"] == 4 and flat["child.scale"] == 3.0 and flat["child.klass"] is Layer
    text = a.debug_string()
    assert "child.dim: 1" in text and "dim: 4" in text
    assert "scale: 1.0" in a.debug_string(omit_default_values={}) and "child.child" not in a.debug_string()


def test_config_for_function_binds_and_validates():
    def fn(a, b=2, *, c=3):
        return a + b * c

    cfg = config_for_function(fn)
    assert cfg.b == 2 and cfg.c == 3 and cfg.a is REQUIRED
    with pytest.raises(config.RequiredFieldMissingError):
        cfg.instantiate()
    assert cfg.set(a=1).instantiate() == 7
    assert cfg.clone(c=1).instantiate() == 3

    def varargs(x, *args, **kwargs):
        return x, args, kwargs

    v = config_for_function(varargs).set(x=1, args=[2, 3], kwargs={"k": 4})
    assert v.instantiate() == (1, (2, 3), {"k": 4})


def test_config_for_class_and_dataclass():
    @dataclasses.dataclass
    class Person:
        name: str
        age: int = 3

    cfg = config_for_class(Person).set(name="x")
    assert cfg.instantiate() == Person("x", 3)
    # A config passed as an argument is handed over as is (the callee decides when to build it).
    def outer(p):
        return p

    o = config_for_function(outer).set(p=cfg)
    assert o.instantiate() == cfg


def test_maybe_set_config_and_similar_names():
    cfg = Layer.default_config()
    maybe_set_config(cfg, dim=3, not_a_field=1)
    assert cfg.dim == 3
    assert config.similar_names("hiden_dim", ["hidden_dim", "input_dim", "x"])[0] == "hidden_dim"


def test_visit_traverses_nested_containers():
    a = Layer.default_config().set(dim=4, child=Layer.default_config().set(dim=1))
    seen = []
    a.visit(visit_fn=lambda k, v: seen.append(k), enter_fn=lambda k, v, default: default)
    assert "child" in seen or any("child" in s for s in seen)
