"""State dicts, msgpack round trips and struct dataclasses."""

import collections
import functools

import numpy as np
import pytest
import torch
from torch.utils import _pytree as pytree

from axlearn_b200.common import serialization, struct

Point = collections.namedtuple("Point", ["x", "y"])


def test_state_dict_round_trip_of_containers():
    target = {"a": [1, (2, 3)], 5: Point(x=1.0, y={"z": 2}), "p": functools.partial(max, 1, key=None)}
    sd = serialization.to_state_dict(target)
    assert sd == {"a": {"0": 1, "1": {"0": 2, "1": 3}}, "5": {"x": 1.0, "y": {"z": 2}},
                  "p": {"args": {"0": 1}, "keywords": {"key": None}}}
    sd["a"]["1"]["0"] = 20
    sd["5"]["y"]["z"] = 7
    restored = serialization.from_state_dict(target, sd)
    assert restored["a"] == [1, (20, 3)] and restored[5] == Point(1.0, {"z": 7}) and restored["p"].func is max
    with pytest.raises(ValueError, match="unique string"):
        serialization.to_state_dict({1: 0, "1": 0})


def test_mismatches_name_the_path():
    target = {"a": {"b": [1, 2]}, "t": Point(1, 2)}
    with pytest.raises(ValueError, match=r"got 2 and 1 at path \./a/b"):
        serialization.from_state_dict(target, {"a": {"b": {"0": 1}}, "t": {"x": 1, "y": 2}})
    with pytest.raises(ValueError, match="not present in state dict at path ./a"):
        serialization.from_state_dict(target, {"a": {}, "t": {"x": 1, "y": 2}})
    with pytest.raises(ValueError, match="named tuple do not match"):
        serialization.from_state_dict(target, {"a": {"b": {"0": 1, "1": 2}}, "t": {"x": 1}})
    with pytest.raises(ValueError, match="already registered"):
        serialization.register_serialization_state(dict, lambda x: x, lambda x, s: s)


def test_msgpack_round_trip():
    tree = {"w": torch.randn(3, 4).to(torch.bfloat16), "i": torch.arange(5), "n": np.arange(6, dtype=np.float64).reshape(2, 3),
            "s": "text", "b": b"\x00\x01", "l": [1, 2.5, None, True], "scalar": np.float32(1.5)}
    blob = serialization.msgpack_serialize(tree)
    back = serialization.from_bytes(tree, blob)
    assert back["w"].dtype == torch.bfloat16 and torch.equal(back["w"], tree["w"]) and torch.equal(back["i"], tree["i"])
    assert isinstance(back["n"], np.ndarray) and (back["n"] == tree["n"]).all()
    assert back["s"] == "text" and back["b"] == b"\x00\x01" and back["l"] == [1, 2.5, None, True] and back["scalar"] == 1.5
    with pytest.raises(TypeError):
        serialization.msgpack_serialize({"x": object()})


@struct.dataclass
class State:
    step: torch.Tensor
    params: dict
    name: str = struct.field(pytree_node=False, default="s")


class Node(struct.PyTreeNode):
    b: int
    a: int


def test_struct_dataclass_is_a_tree_and_serialises():
    s = State(step=torch.tensor(3), params={"w": torch.ones(2)})
    leaves, spec = pytree.tree_flatten(s)
    assert len(leaves) == 2 and torch.equal(leaves[0], torch.ones(2))           # fields in name order: params, step
    doubled = pytree.tree_map(lambda t: t * 2, s)
    assert isinstance(doubled, State) and doubled.step.item() == 6 and doubled.name == "s"
    assert pytree.tree_unflatten(leaves, spec).name == "s"
    with pytest.raises(Exception):
        s.step = 1                                                               # frozen
    assert s.replace(name="t").name == "t"
    sd = serialization.to_state_dict(s)
    assert set(sd) == {"step", "params"} and set(sd["params"]) == {"w"}
    sd["step"] = torch.tensor(9)
    assert serialization.from_state_dict(s, sd).step.item() == 9
    with pytest.raises(ValueError, match="Missing field step"):
        serialization.from_state_dict(s, {"params": {"w": 1}})
    with pytest.raises(ValueError, match="Unknown field"):
        serialization.from_state_dict(s, {"params": {"w": 1}, "step": 1, "extra": 2})
    back = serialization.from_bytes(s, serialization.msgpack_serialize(s))
    assert back.step.item() == 3 and torch.equal(back.params["w"], torch.ones(2))
    n = Node(b=1, a=2)
    assert pytree.tree_leaves(n) == [2, 1] and n.replace(a=5).a == 5
    assert struct.dataclass(State) is State
