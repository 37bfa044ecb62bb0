"""State dicts of nested containers (reference: axlearn/common/serialization.py:17-199), plus a
compact binary form.

``to_state_dict`` turns dicts, lists, tuples, named tuples and registered classes into nested
dicts with STRING keys (a list becomes ``{"0": ..., "1": ...}``); ``from_state_dict`` restores a
state dict into the structure of a target, reporting the path of a mismatch.  Other types register
a pair of functions with ``register_serialization_state`` (``common/struct.py`` does so for its
dataclasses).

``msgpack_serialize`` / ``msgpack_restore`` write a state dict whose leaves are tensors, NumPy
arrays, scalars, strings or bytes as one msgpack blob: tensors and arrays travel as an extension
type holding dtype, shape and raw bytes (bfloat16 is kept bit-exactly as 16-bit words).
"""

from __future__ import annotations

import contextlib
import functools
import threading
from typing import Any, Callable

import numpy as np
import torch

_STATE_DICT_REGISTRY: dict[Any, Any] = {}


class _ErrorContext(threading.local):
    def __init__(self):
        super().__init__()
        self.path: list[str] = []


_error_context = _ErrorContext()


@contextlib.contextmanager
def _record_path(name: str):
    try:
        _error_context.path.append(name)
        yield
    finally:
        _error_context.path.pop()


def current_path() -> str:
    """The path within the state dict at which ``from_state_dict`` currently is (for messages)."""
    return "/".join(_error_context.path)


class _NamedTuple:
    """Registry key under which every named tuple type is handled."""


def _is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(x, "_fields")


def _registry_type(target: Any) -> Any:
    return _NamedTuple if _is_namedtuple(target) else type(target)


def to_state_dict(target: Any) -> Any:
    ty = _registry_type(target)
    if ty not in _STATE_DICT_REGISTRY:
        return target
    state = _STATE_DICT_REGISTRY[ty][0](target)
    if isinstance(state, dict):
        for key in state:
            if not isinstance(key, str):
                raise ValueError(f"A state dict must only have string keys. Instead, encountered key {key} of type {type(key)}.")
    return state


def from_state_dict(target: Any, state: Any, name: str = ".") -> Any:
    """A copy of ``target`` with the values of ``state``; unregistered targets are replaced by the
    state as it is."""
    ty = _registry_type(target)
    if ty not in _STATE_DICT_REGISTRY:
        return state
    with _record_path(name):
        return _STATE_DICT_REGISTRY[ty][1](target, state)


def register_serialization_state(ty: type, ty_to_state_dict: Callable, ty_from_state_dict: Callable,
                                 override: bool = False) -> None:
    if ty in _STATE_DICT_REGISTRY and not override:
        raise ValueError(f'A serialization handler for "{ty.__name__}" is already registered.')
    _STATE_DICT_REGISTRY[ty] = (ty_to_state_dict, ty_from_state_dict)


def _list_state_dict(xs) -> dict:
    return {str(i): to_state_dict(x) for i, x in enumerate(xs)}


def _restore_list(xs, state_dict: dict) -> list:
    if len(state_dict) != len(xs):
        raise ValueError("The size of the list and the state dict do not match, "
                         f"got {len(xs)} and {len(state_dict)} at path {current_path()}")
    return [from_state_dict(xs[i], state_dict[str(i)], name=str(i)) for i in range(len(xs))]


def _dict_state_dict(xs: dict) -> dict:
    str_keys = {str(k) for k in xs}
    if len(str_keys) != len(xs):
        raise ValueError(f"Dict keys do not have a unique string representation: {str_keys} vs given: {xs}")
    return {str(k): to_state_dict(v) for k, v in xs.items()}


def _restore_dict(xs: dict, state_dict: dict) -> dict:
    diff = {str(k) for k in xs}.difference(state_dict.keys())
    if diff:
        raise ValueError("The target dict keys and state dict keys do not match, target dict contains keys "
                         f"{diff} which are not present in state dict at path {current_path()}")
    return {k: from_state_dict(v, state_dict[str(k)], name=str(k)) for k, v in xs.items()}


def _namedtuple_state_dict(xs) -> dict:
    return {k: to_state_dict(getattr(xs, k)) for k in xs._fields}


def _restore_namedtuple(xs, state_dict: dict):
    if set(state_dict) != set(xs._fields):
        raise ValueError("The field names of the state dict and the named tuple do not match, "
                         f"got {set(state_dict)} and {set(xs._fields)} at path {current_path()}")
    return type(xs)(**{k: from_state_dict(getattr(xs, k), v, name=k) for k, v in state_dict.items()})


register_serialization_state(dict, _dict_state_dict, _restore_dict)
register_serialization_state(list, _list_state_dict, _restore_list)
register_serialization_state(tuple, _list_state_dict, lambda xs, sd: tuple(_restore_list(list(xs), sd)))
register_serialization_state(_NamedTuple, _namedtuple_state_dict, _restore_namedtuple)
register_serialization_state(
    functools.partial,
    lambda x: {"args": to_state_dict(x.args), "keywords": to_state_dict(x.keywords)},
    lambda x, sd: functools.partial(x.func, *from_state_dict(x.args, sd["args"]),
                                    **from_state_dict(x.keywords, sd["keywords"])))


# ------------------------------------------------------------------------------------------------
# Binary form.

_EXT_NDARRAY, _EXT_TENSOR = 1, 2


def _pack_array(a: np.ndarray) -> bytes:
    import msgpack

    return msgpack.packb((a.dtype.str, list(a.shape), np.ascontiguousarray(a).tobytes()), use_bin_type=True)


def _default(obj: Any):
    import msgpack

    if isinstance(obj, torch.Tensor):
        t = obj.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            payload = msgpack.packb(("bfloat16", list(t.shape), t.view(torch.int16).numpy().tobytes()), use_bin_type=True)
        else:
            payload = _pack_array(t.numpy())
        return msgpack.ExtType(_EXT_TENSOR, payload)
    if isinstance(obj, np.ndarray):
        return msgpack.ExtType(_EXT_NDARRAY, _pack_array(obj))
    if isinstance(obj, np.generic):
        return obj.item()
    raise TypeError(f"cannot serialise {type(obj)}")


def _ext_hook(code: int, data: bytes):
    import msgpack

    if code not in (_EXT_NDARRAY, _EXT_TENSOR):
        return msgpack.ExtType(code, data)
    dtype, shape, raw = msgpack.unpackb(data, raw=False)
    if dtype == "bfloat16":
        return torch.from_numpy(np.frombuffer(raw, dtype=np.int16).reshape(shape).copy()).view(torch.bfloat16)
    arr = np.frombuffer(raw, dtype=np.dtype(dtype)).reshape(shape).copy()
    return torch.from_numpy(arr) if code == _EXT_TENSOR else arr


def msgpack_serialize(target: Any) -> bytes:
    """``to_state_dict(target)`` as one msgpack blob."""
    import msgpack

    return msgpack.packb(to_state_dict(target), default=_default, use_bin_type=True)


def msgpack_restore(data: bytes) -> Any:
    import msgpack

    return msgpack.unpackb(data, ext_hook=_ext_hook, raw=False, strict_map_key=False)


def from_bytes(target: Any, data: bytes) -> Any:
    """Restores ``data`` into the structure of ``target``."""
    return from_state_dict(target, msgpack_restore(data))
