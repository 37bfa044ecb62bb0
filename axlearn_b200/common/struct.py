"""Frozen dataclasses that are trees (reference: axlearn/common/flax_struct.py:26-145).

``@struct.dataclass`` makes a frozen dataclass whose fields are tree children unless declared with
``field(pytree_node=False)`` (static metadata).  Such a class

* flattens with ``torch.utils._pytree`` (children in ascending field-name order by default), so
  ``tree_map`` and this framework's tree utilities walk through it;
* has a ``replace(**updates)`` method;
* takes part in ``serialization.to_state_dict`` / ``from_state_dict`` with its tree fields.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Optional, TypeVar

from torch.utils import _pytree as pytree

from axlearn_b200.common import serialization

_T = TypeVar("_T")


def field(pytree_node: bool = True, **kwargs):
    return dataclasses.field(metadata={"pytree_node": pytree_node}, **kwargs)  # pylint: disable=invalid-field-call


def dataclass(klass: Optional[_T] = None, *, flatten_order: Optional[str] = "asc", **kwargs) -> _T:
    if klass is None:
        return lambda k: dataclass(k, flatten_order=flatten_order, **kwargs)
    if "_axlearn_dataclass" in klass.__dict__:
        return klass
    kwargs.setdefault("frozen", True)
    dataklass = dataclasses.dataclass(**kwargs)(klass)
    fields = list(dataclasses.fields(dataklass))
    if flatten_order == "asc":
        fields.sort(key=lambda f: f.name)
    elif flatten_order is not None:
        raise NotImplementedError(flatten_order)
    data_fields = [f.name for f in fields if f.init and f.metadata.get("pytree_node", True)]
    meta_fields = [f.name for f in fields if f.init and not f.metadata.get("pytree_node", True)]

    def replace(self, **updates):
        return dataclasses.replace(self, **updates)

    dataklass.replace = replace

    def flatten(x):
        return [getattr(x, n) for n in data_fields], tuple(getattr(x, n) for n in meta_fields)

    def unflatten(children, meta):
        return dataklass(**dict(zip(data_fields, children)), **dict(zip(meta_fields, meta)))

    def flatten_with_keys(x):
        return [(pytree.GetAttrKey(n), getattr(x, n)) for n in data_fields], tuple(getattr(x, n) for n in meta_fields)

    pytree.register_pytree_node(dataklass, flatten, unflatten, flatten_with_keys_fn=flatten_with_keys,
                                serialized_type_name=f"{dataklass.__module__}.{dataklass.__qualname__}")

    def to_state_dict(x):
        return {n: serialization.to_state_dict(getattr(x, n)) for n in data_fields}

    def from_state_dict(x, state):
        state = dict(state)
        updates = {}
        for n in data_fields:
            if n not in state:
                raise ValueError(f"Missing field {n} in state dict while restoring an instance of "
                                 f"{dataklass.__name__}, at path {serialization.current_path()}")
            updates[n] = serialization.from_state_dict(getattr(x, n), state.pop(n), name=n)
        if state:
            raise ValueError(f'Unknown field(s) "{", ".join(state)}" in state dict while restoring an instance of '
                             f"{dataklass.__name__} at path {serialization.current_path()}")
        return x.replace(**updates)

    serialization.register_serialization_state(dataklass, to_state_dict, from_state_dict)
    dataklass._axlearn_dataclass = True  # pylint: disable=protected-access
    return dataklass


class PyTreeNode:
    """Base class form of ``@dataclass``: subclasses become struct dataclasses."""

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        dataclass(cls)

    def replace(self: _T, **overrides) -> _T:  # replaced by ``dataclass``
        raise NotImplementedError

    def __init__(self, *args: Any, **kwargs: Any):  # replaced by ``dataclass``
        raise NotImplementedError
