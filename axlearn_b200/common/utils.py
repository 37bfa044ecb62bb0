"""Tree, dtype, regex-rule and miscellaneous helpers shared by every layer of the stack.

A "tree" is any nesting of dict / list / tuple / NamedTuple with tensor (or arbitrary)
leaves.  Paths join keys with ``/``; dict keys are visited in sorted order, sequences by
index, NamedTuples by field name — the same convention the reference uses to name
checkpoint tensors (axlearn/common/utils.py:377-431).

Parity targets in the reference (axlearn/common/utils.py): ``TensorSpec`` (:127),
``flatten_items``/``tree_paths`` (:396-431), ``VDict`` (:433), ``split_prng_key`` (:539),
``cast_floats`` (:1246), ``count_model_params`` (:1438), ``prune_tree``/``prune_empty``
(:1534-1620), data-dir stack (:1621-1670), ``match_regex_rules`` (:1679),
``thread_stack_traces`` (:2028), ``find_cycles`` (:2067), ``sequence_mask`` (:2130),
``replace_layer_config_recursively`` (:2206).  Mesh helpers live in
``axlearn_b200.parallel.mesh``.
"""

from __future__ import annotations

import contextlib
import dataclasses
import re
import sys
import threading
import traceback
from typing import Any, Callable, NamedTuple, Optional, Sequence, Union

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.config import ConfigBase, InstantiableConfig, similar_names

Tensor = torch.Tensor
Nested = Any
NestedTensor = Any


# --------------------------------------------------------------------------------------
# Partition / tensor specs.
# --------------------------------------------------------------------------------------


class PartitionSpec(tuple):
    """Per-dimension mesh axis names: each entry is ``None``, an axis name, or a tuple of
    axis names (the dimension is split over their product, major to minor)."""

    def __new__(cls, *axes):
        return super().__new__(cls, axes)

    def __repr__(self):
        return f"PartitionSpec{tuple(self)!r}"

    def __reduce__(self):
        return (_rebuild_pspec, (tuple(self),))


def _rebuild_pspec(axes):
    return PartitionSpec(*axes)


@dataclasses.dataclass
class TensorSpec:
    """Shape / dtype / sharding of a tensor that may not exist yet."""

    shape: Sequence[int]
    dtype: Optional[torch.dtype] = None
    mesh_axes: Optional[Sequence[Any]] = None

    __config_value__ = True


# --------------------------------------------------------------------------------------
# Tree utilities.
# --------------------------------------------------------------------------------------


def _is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(type(x), "_fields")


def _children(tree: Any) -> Optional[list[tuple[str, Any]]]:
    if isinstance(tree, dict):
        keys = list(tree.keys())
        try:
            keys = sorted(keys)
        except TypeError:
            pass
        return [(str(k), tree[k]) for k in keys]
    if _is_namedtuple(tree):
        return [(f, getattr(tree, f)) for f in tree._fields]
    if isinstance(tree, (list, tuple)):
        return [(str(i), v) for i, v in enumerate(tree)]
    if dataclasses.is_dataclass(tree) and not isinstance(tree, type) and getattr(
        tree, "__tree_node__", False
    ):
        return [(f.name, getattr(tree, f.name)) for f in dataclasses.fields(tree)]
    return None


def flatten_items(
    tree: Nested, *, separator: str = "/", is_leaf: Optional[Callable[[Any], bool]] = None
) -> list[tuple[str, Any]]:
    """``[(path, leaf), ...]`` in deterministic order. ``None`` subtrees are skipped."""
    out: list[tuple[str, Any]] = []

    def walk(prefix: str, node: Any):
        if node is None:
            return
        kids = None if (is_leaf is not None and is_leaf(node)) else _children(node)
        if kids is None:
            out.append((prefix, node))
            return
        for k, v in kids:
            walk(f"{prefix}{separator}{k}" if prefix else k, v)

    walk("", tree)
    return out


def tree_leaves(tree: Nested, *, is_leaf=None) -> list[Any]:
    return [v for _, v in flatten_items(tree, is_leaf=is_leaf)]


def tree_map(fn: Callable, tree: Nested, *rest: Nested, is_leaf=None) -> Nested:
    """Maps ``fn`` over corresponding leaves; container types (incl. VDict, NamedTuple) are
    preserved.  ``None`` is treated as an empty subtree."""

    def walk(node: Any, *others: Any):
        if node is None:
            return None
        if is_leaf is not None and is_leaf(node):
            return fn(node, *others)
        if isinstance(node, dict):
            return type(node)((k, walk(v, *[o[k] for o in others])) for k, v in node.items())
        if _is_namedtuple(node):
            return type(node)(*[walk(v, *[o[i] for o in others]) for i, v in enumerate(node)])
        if isinstance(node, (list, tuple)):
            return type(node)(walk(v, *[o[i] for o in others]) for i, v in enumerate(node))
        if dataclasses.is_dataclass(node) and not isinstance(node, type) and getattr(
            node, "__tree_node__", False
        ):
            return dataclasses.replace(
                node,
                **{
                    f.name: walk(getattr(node, f.name), *[getattr(o, f.name) for o in others])
                    for f in dataclasses.fields(node)
                },
            )
        return fn(node, *others)

    return walk(tree, *rest)


def tree_paths(tree: Nested, *, separator: str = "/", is_leaf=None) -> Nested:
    """A tree of the same structure whose leaves are their own paths."""

    def walk(prefix: str, node: Any):
        if node is None:
            return None
        join = lambda k: f"{prefix}{separator}{k}" if prefix else str(k)
        if is_leaf is not None and is_leaf(node):
            return prefix
        if isinstance(node, dict):
            return type(node)((k, walk(join(k), v)) for k, v in node.items())
        if _is_namedtuple(node):
            return type(node)(*[walk(join(f), getattr(node, f)) for f in node._fields])
        if isinstance(node, (list, tuple)):
            return type(node)(walk(join(i), v) for i, v in enumerate(node))
        return prefix

    return walk("", tree)


def get_recursively(tree: Nested, path: Union[str, Sequence[str]], separator: str = "/") -> Any:
    if isinstance(path, str):
        path = path.split(separator) if path else []
    cur = tree
    for k in path:
        if isinstance(cur, dict):
            if k not in cur:
                raise KeyError(f"No key {k!r} in path {path}")
            cur = cur[k]
        elif _is_namedtuple(cur) and k in cur._fields:
            cur = getattr(cur, k)
        elif isinstance(cur, (list, tuple)):
            cur = cur[int(k)]
        else:
            raise KeyError(f"Cannot descend into {type(cur)} with key {k!r}")
    return cur


def set_recursively(
    tree: dict, *, value: Any, path: Union[str, Sequence[str]], separator: str = "/"
) -> None:
    if isinstance(path, str):
        path = path.split(separator)
    if not path:
        raise ValueError("path must not be empty")
    cur = tree
    for k in path[:-1]:
        cur = cur.setdefault(k, {})
    cur[path[-1]] = value


def unflatten_items(items: Sequence[tuple[str, Any]], separator: str = "/") -> dict:
    out: dict = {}
    for path, v in items:
        set_recursively(out, value=v, path=path, separator=separator)
    return out


class VDict(dict):
    """A dict whose leaves carry an extra leading "vectorised" dim (e.g. stacked per-layer
    parameters).  Keys iterate in sorted order."""

    def __repr__(self):
        return f"VDict({dict.__repr__(self)})"

    def items(self):
        return [(k, self[k]) for k in sorted(self.keys())]


def vectorized_tree_map(fn: Callable, tree: Nested) -> Nested:
    """``tree_map`` that applies ``fn`` per index of the leading dim for leaves under a VDict
    (reference: axlearn/common/utils.py ``vectorized_tree_map``), so that ``fn`` always sees
    the per-layer shape (e.g. batch-leading cache tensors of stacked layers)."""

    def walk(node, depth):
        if node is None:
            return None
        if isinstance(node, dict):
            d = depth + 1 if isinstance(node, VDict) else depth
            return type(node)((k, walk(v, d)) for k, v in node.items())
        if _is_namedtuple(node):
            return type(node)(*[walk(v, depth) for v in node])
        if isinstance(node, (list, tuple)):
            return type(node)(walk(v, depth) for v in node)
        return apply(node, depth)

    def apply(x, depth):
        if depth == 0 or not isinstance(x, torch.Tensor):
            return fn(x)
        return torch.stack([apply(x[i], depth - 1) for i in range(x.shape[0])], dim=0)

    return walk(tree, 0)


def expand_vdicts(tree: Nested) -> Nested:
    """Replaces every VDict by a list of per-index plain dicts."""

    def expand(node):
        if isinstance(node, VDict):
            leaves = tree_leaves(dict(node))
            n = leaves[0].shape[0] if leaves else 0
            return [expand(tree_map(lambda t, i=i: t[i], dict(node))) for i in range(n)]
        if isinstance(node, dict):
            return {k: expand(v) for k, v in node.items()}
        return node

    return expand(tree)


def prune_tree(
    tree: Nested, should_prune: Callable[[str, Any], bool], *, prefix: str = "", separator="/"
) -> Nested:
    """Removes dict entries for which ``should_prune(path, value)`` holds."""
    if isinstance(tree, dict) and should_prune(prefix, tree):
        return {}
    if not isinstance(tree, dict):
        return tree
    out = type(tree)()
    for k, v in tree.items():
        path = f"{prefix}{separator}{k}" if prefix else str(k)
        if should_prune(path, v):
            continue
        out[k] = prune_tree(v, should_prune, prefix=path, separator=separator)
    return out


def prune_empty(tree: Nested) -> Nested:
    """Drops empty dicts (recursively)."""
    if not isinstance(tree, dict):
        return tree
    out = type(tree)()
    for k, v in tree.items():
        v = prune_empty(v)
        if isinstance(v, dict) and not v:
            continue
        out[k] = v
    return out


def tree_merge(primary: Nested, secondary: Nested, *, leaf_merge_fn=None) -> Nested:
    """Union of two dict trees; on leaf conflict ``leaf_merge_fn(primary, secondary)``."""
    if isinstance(primary, dict) and isinstance(secondary, dict):
        out = type(primary)(primary)
        for k, v in secondary.items():
            out[k] = tree_merge(primary[k], v, leaf_merge_fn=leaf_merge_fn) if k in primary else v
        return out
    if isinstance(primary, dict) and not primary:
        return secondary
    if isinstance(secondary, dict) and not secondary:
        return primary
    if leaf_merge_fn is None:
        raise ValueError(f"Conflicting leaves: {primary!r} vs {secondary!r}")
    return leaf_merge_fn(primary, secondary)


def match_regex_rules(
    x: str, *, rules: Sequence[tuple[str, Any]], default_value: Any = None
) -> Any:
    """Value of the first rule whose regex fully matches ``x``."""
    for regex, value in rules:
        if re.fullmatch(regex, x):
            return value
    return default_value


# --------------------------------------------------------------------------------------
# Dtype helpers.
# --------------------------------------------------------------------------------------

_FLOAT_DTYPES = (torch.float32, torch.bfloat16, torch.float16, torch.float64)


def cast_floats(tree: NestedTensor, to_dtype: Optional[torch.dtype]) -> NestedTensor:
    """Casts floating-point leaves to ``to_dtype``; other leaves pass through."""
    if to_dtype is None:
        return tree

    def cast(x):
        if isinstance(x, torch.Tensor) and x.dtype in _FLOAT_DTYPES and x.dtype != to_dtype:
            return x.to(to_dtype)
        return x

    return tree_map(cast, tree)


def per_param_dtype_by_path(
    default_dtype: Optional[torch.dtype] = None,
    *,
    update_rules: Optional[Sequence[tuple[str, Optional[torch.dtype]]]] = None,
) -> Callable[[NestedTensor], NestedTensor]:
    """Returns ``tree -> tree of dtypes`` choosing a dtype per parameter path."""

    def fn(tree):
        def pick(path):
            return match_regex_rules(path, rules=update_rules or (), default_value=default_dtype)

        return tree_map(pick, tree_paths(tree))

    return fn


def cast_floats_per_param(tree: NestedTensor, dtypes: Nested) -> NestedTensor:
    def cast(x, dt):
        if isinstance(x, torch.Tensor) and dt is not None and x.dtype in _FLOAT_DTYPES:
            return x.to(dt)
        return x

    return tree_map(cast, tree, dtypes)


def count_model_params(tree: NestedTensor) -> int:
    return sum(int(x.numel()) for x in tree_leaves(tree) if hasattr(x, "numel"))


def split_prng_key(key: torch.Tensor, num_keys: Union[int, Sequence[int]]) -> list:
    """Splits into ``num_keys`` keys (nested lists for a shape tuple)."""
    if isinstance(num_keys, int):
        return prng.split(key, num_keys)
    shape = tuple(num_keys)
    total = 1
    for s in shape:
        total *= s
    flat = prng.split(key, total)

    def build(dims, offset):
        if len(dims) == 1:
            return flat[offset : offset + dims[0]]
        stride = 1
        for d in dims[1:]:
            stride *= d
        return [build(dims[1:], offset + i * stride) for i in range(dims[0])]

    return build(shape, 0)


def sequence_mask(*, lengths: Tensor, max_len: int, dtype=torch.int32) -> Tensor:
    """``mask[..., t] = t < lengths[...]``."""
    ar = torch.arange(max_len, device=lengths.device)
    return (ar < lengths.unsqueeze(-1)).to(dtype)


def safe_not(mask: Tensor) -> Tensor:
    return ~(mask.to(torch.bool))


# --------------------------------------------------------------------------------------
# Data-dir stack.
# --------------------------------------------------------------------------------------

_data_dir = threading.local()


@contextlib.contextmanager
def set_data_dir(data_dir: Optional[str]):
    """Scopes the dataset root; ``"FAKE"`` selects synthetic data in input configs."""
    stack = getattr(_data_dir, "stack", None)
    if stack is None:
        stack = _data_dir.stack = []
    if stack and stack[-1] not in (None, "FAKE") and data_dir != stack[-1]:
        raise ValueError(f"data_dir already set to {stack[-1]}")
    stack.append(data_dir)
    try:
        yield
    finally:
        stack.pop()


def get_data_dir() -> Optional[str]:
    stack = getattr(_data_dir, "stack", None)
    return stack[-1] if stack else None


def get_or_none(tree: Optional[dict], key: str) -> Any:
    return None if tree is None else tree.get(key)


# --------------------------------------------------------------------------------------
# Debugging helpers.
# --------------------------------------------------------------------------------------


def thread_stack_traces() -> list[list[str]]:
    """Stack traces of all live Python threads (used by the trainer watchdog)."""
    out = []
    frames = sys._current_frames()  # pylint: disable=protected-access
    for t in threading.enumerate():
        frame = frames.get(t.ident)
        if frame is None:
            continue
        lines = [f"Thread: {t.name} ({t.ident})"]
        lines.extend(l.rstrip("\n") for l in traceback.format_stack(frame))
        out.append(lines)
    return out


def find_cycles(graph: dict[Any, Sequence[Any]]) -> Optional[list[Any]]:
    """Returns one cycle (as a node list) of a directed graph, or None."""
    WHITE, GREY, BLACK = 0, 1, 2
    colour = {n: WHITE for n in graph}
    stack: list[Any] = []

    def dfs(n) -> Optional[list[Any]]:
        colour[n] = GREY
        stack.append(n)
        for m in graph.get(n, ()):
            c = colour.get(m, WHITE)
            if c == GREY:
                return stack[stack.index(m) :] + [m]
            if c == WHITE:
                colour.setdefault(m, WHITE)
                found = dfs(m)
                if found:
                    return found
        stack.pop()
        colour[n] = BLACK
        return None

    for node in list(graph):
        if colour[node] == WHITE:
            found = dfs(node)
            if found:
                return found
    return None


def raise_for_cycles(graph: dict[Any, Sequence[Any]]) -> None:
    cyc = find_cycles(graph)
    if cyc:
        raise ValueError(f"Circular reference: {' -> '.join(map(str, cyc))}")


def replace_layer_config_recursively(
    cfg: ConfigBase,
    *,
    target_cls: type,
    source_config: InstantiableConfig,
    exclude_keys: Sequence[str] = ("name",),
) -> int:
    """Replaces every sub-config whose ``klass`` is ``target_cls`` by ``source_config``,
    carrying over fields the two share (except ``exclude_keys``... which are kept from the
    original).  Returns the number of replacements."""
    count = 0

    def visit(node: Any) -> Any:
        nonlocal count
        if isinstance(node, ConfigBase):
            if "klass" in node and node.klass is target_cls:
                new = source_config.clone()
                for k, v in node.items():
                    if k == "klass":
                        continue
                    if k in new and (k in exclude_keys or k not in ("klass",)):
                        if k in exclude_keys or getattr(new, k) is None:
                            setattr(new, k, v)
                count += 1
                return new
            for k, v in node.items():
                nv = visit(v)
                if nv is not v:
                    setattr(node, k, nv)
            return node
        if isinstance(node, list):
            for i, v in enumerate(node):
                node[i] = visit(v)
            return node
        if isinstance(node, dict):
            for k in list(node):
                node[k] = visit(node[k])
            return node
        return node

    visit(cfg)
    return count


_per_param_settings: dict[str, dict[str, Any]] = {}


def register_per_param_settings(settings: Nested, *, description: str) -> Nested:
    """Records per-parameter settings (e.g. weight-decay scales) for golden tests."""
    _per_param_settings[description] = dict(flatten_items(settings))
    return settings


def get_per_param_settings() -> dict[str, dict[str, Any]]:
    return _per_param_settings


class StackedKeyArray(NamedTuple):
    """A list of keys treated as one leaf (for vectorised initialisation)."""

    keys: list


__all__ = [n for n in dir() if not n.startswith("_")]
