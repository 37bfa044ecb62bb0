"""Module tree and invocation contexts.

A ``Module`` is a stateless node of a named tree.  All mutable things that a call needs —
the parameter/state sub-tree, the PRNG key, the training flag and the collection that
receives summaries / state updates / module outputs — travel in an ``InvocationContext``.
Calling a public method of a child module from inside a parent's method transparently
pushes the child's context (state slice ``parent.state[child.name]``, key
``fold_in(parent_key, hash(child.name))``, child output collection), so user code reads like
ordinary object-oriented code while staying functional.

``functional(module, ...)`` is the only entry point from "outside": it builds the root
context, runs a method and returns ``(outputs, OutputCollection)``.

Parity targets in the reference (axlearn/common/module.py): ``OutputCollection`` (:251),
``InvocationContext`` (:376), context stack (:563-655), ``child_context`` (:646), method
wrapping (:738-885), ``Module`` (:781), ``_add_child`` (:944), shared modules (:1004-1091),
``functional`` (:1212), ``scan_in_context`` (:1279), ``nowrap`` (:184).

Differences by design: tensors are ``torch.Tensor``; PRNG keys are 128-bit host-side values
(see ``prng.py``); ``scan_in_context`` is a Python loop (there is no tracing compiler — the
launch-bound inner loops are captured in CUDA graphs by the callers that need it), and every
wrapped call opens an NVTX range named ``name[Class]`` when profiling is enabled.
"""

from __future__ import annotations

import contextlib
import dataclasses
import functools
import hashlib
import re
import threading
from typing import Any, Callable, NamedTuple, Optional, Sequence, TypeVar, Union

import torch

from axlearn_b200.common import prng
from axlearn_b200.common import debug_utils, traceback_util
from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class

NestedTensor = Union[torch.Tensor, dict[str, Any]]
Tensor = torch.Tensor
M = TypeVar("M", bound="Module")

_NAME_RE = re.compile(r"^[a-zA-Z][a-zA-Z0-9_]*$")


def nowrap(fn: Callable) -> Callable:
    """Marks a public method as context-free: it is *not* wrapped, so it can be called
    outside an invocation context (e.g. pure shape helpers)."""
    fn.__nowrap__ = True
    return fn


# --------------------------------------------------------------------------------------
# Output collection.
# --------------------------------------------------------------------------------------


class OutputCollection(NamedTuple):
    """Side outputs of a call, each a nested dict mirroring the module tree."""

    summaries: dict
    state_updates: dict
    module_outputs: dict

    def add_child(self, name: str) -> "OutputCollection":
        if not _NAME_RE.fullmatch(name):
            raise ValueError(f'Invalid child name "{name}"')
        kids = []
        for coll in self:
            if name in coll:
                raise ValueError(f'Output collection already has a child named "{name}"')
            coll[name] = {}
            kids.append(coll[name])
        return OutputCollection(*kids)

    def get_or_add_child(self, name: str) -> "OutputCollection":
        return OutputCollection(*[coll.setdefault(name, {}) for coll in self])

    def update(self, other: "OutputCollection") -> None:
        for mine, theirs in zip(self, other):
            mine.update(theirs)


def new_output_collection() -> OutputCollection:
    return OutputCollection(summaries={}, state_updates={}, module_outputs={})


def propagate_repeated_output_collections(
    per_iter: Sequence[OutputCollection],
    *,
    child_name_prefix: str,
    target: OutputCollection,
) -> None:
    """Files each iteration's collection under ``{prefix}{i}`` in ``target``.

    ``state_updates`` of a repeated body are not representable per iteration and must be
    empty (same restriction as the reference's scan)."""
    for i, coll in enumerate(per_iter):
        if coll.state_updates:
            raise NotImplementedError("state_updates inside a repeated body are not supported")
        child = target.get_or_add_child(f"{child_name_prefix}{i}")
        child.summaries.update(coll.summaries)
        child.module_outputs.update(coll.module_outputs)


# --------------------------------------------------------------------------------------
# Invocation context.
# --------------------------------------------------------------------------------------


@dataclasses.dataclass
class InvocationContext:
    name: str
    parent: Optional["InvocationContext"]
    module: "Module"
    state: Any  # Nested dict of tensors for ``module``.
    is_training: bool
    prng_key: Optional[torch.Tensor]
    output_collection: OutputCollection

    def path(self) -> str:
        if self.parent is None:
            return self.name
        return f"{self.parent.path()}.{self.name}"

    def add_child(self, name: str, **overrides) -> "InvocationContext":
        """Context of child module ``name`` derived from this one."""
        if "module" in overrides:
            # A named sub-invocation of a given module (e.g. the same tower run once per input
            # field): outputs and PRNG keys are scoped by ``name``; when the module is this
            # context's own, it keeps this context's state.
            child_module = overrides["module"]
            if "state" not in overrides:
                if child_module is self.module:
                    overrides = dict(overrides, state=self.state)
                else:  # a child invoked under another name keeps its own state
                    for child_name, child in self.module._children.items():  # pylint: disable=protected-access
                        if child is child_module and isinstance(self.state, dict):
                            overrides = dict(overrides, state=self.state.get(child_name, {}))
                            break
        else:
            child_module = self.module._children[name]  # pylint: disable=protected-access
        kwargs: dict[str, Any] = dict(
            name=name, parent=self, module=child_module, is_training=self.is_training
        )
        if "state" not in overrides:
            st = self.state
            kwargs["state"] = st.get(name, {}) if isinstance(st, dict) else {}
        if "prng_key" not in overrides:
            kwargs["prng_key"] = (
                None if self.prng_key is None else prng.fold_in(self.prng_key, _name_hash(name))
            )
        if "output_collection" not in overrides:
            kwargs["output_collection"] = self.output_collection.get_or_add_child(name)
        kwargs.update(overrides)
        return InvocationContext(**kwargs)

    def add_summary(self, name: str, value: Any) -> None:
        self.output_collection.summaries[name] = value

    def add_state_update(self, name: str, value: Any) -> None:
        self.output_collection.state_updates[name] = value

    def add_module_output(self, name: str, value: Any) -> None:
        self.output_collection.module_outputs[name] = value

    def set_state_update(self, value: Any) -> None:
        """Replaces the whole state-update subtree of this module."""
        if self.parent is None:
            raise ValueError("Cannot replace state updates of the root context")
        self.parent.output_collection.state_updates[self.name] = value

    def get_module_outputs(self) -> dict:
        return self.output_collection.module_outputs

    def functional(self, method_fn: Callable) -> Callable:
        """Runs ``method_fn`` in a *copy* of this context with a fresh output collection;
        returns ``(outputs, output_collection)`` and leaves this context untouched."""

        def call(*args, **kwargs):
            ctx = dataclasses.replace(self, output_collection=new_output_collection())
            with set_current_context(ctx, require_parent=False):
                out = method_fn(*args, **kwargs)
            return out, ctx.output_collection

        return call


def _name_hash(name: str) -> int:
    return int(hashlib.md5(name.encode()).hexdigest(), 16) % (2**31 - 1)


class _Stack(threading.local):
    def __init__(self):
        self.stack: list[InvocationContext] = []


_tls = _Stack()


def current_context() -> Optional[InvocationContext]:
    return _tls.stack[-1] if _tls.stack else None


def clone_context_stack() -> list[InvocationContext]:
    """Snapshot of this thread's stack, for handing to a worker thread."""
    return list(_tls.stack)


def install_context_stack(stack: list[InvocationContext]) -> None:
    if _tls.stack:
        raise ValueError("A context stack is already installed in this thread")
    _tls.stack = list(stack)


@contextlib.contextmanager
def set_current_context(ctx: InvocationContext, *, require_parent: bool = True):
    cur = current_context()
    if require_parent and cur is not None and ctx.parent is not cur and ctx is not cur:
        # Allowed but unusual: calling across the tree (shared modules do this).
        pass
    _tls.stack.append(ctx)
    try:
        yield ctx
    finally:
        _tls.stack.pop()


@contextlib.contextmanager
def child_context(name: str, **overrides):
    """Enters the context of child ``name`` of the current module."""
    cur = current_context()
    if cur is None:
        raise RuntimeError("child_context() called outside an invocation context")
    with set_current_context(cur.add_child(name, **overrides)) as ctx:
        yield ctx


_nvtx_enabled = False


def enable_nvtx_ranges(flag: bool = True) -> None:
    """When on, every wrapped module call is bracketed by an NVTX range ``name[Class]`` so
    that kernel timelines carry the module path."""
    global _nvtx_enabled
    _nvtx_enabled = flag


def _wrap_method(fn: Callable) -> Callable:
    @functools.wraps(fn)
    def wrapped(self: "Module", *args, **kwargs):
        ctx = current_context()
        if ctx is None or ctx.module is self:
            if ctx is None and not getattr(self, "_allow_contextless", False):
                raise RuntimeError(
                    f"{type(self).__name__}.{fn.__name__}() needs an invocation context; "
                    "call it through functional() or from a parent module's method"
                )
            return fn(self, *args, **kwargs)
        target = self._resolve_context(ctx)  # pylint: disable=protected-access
        if _nvtx_enabled and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(f"{self.name}[{type(self).__name__}]")
            try:
                with set_current_context(target):
                    return self._call_in_context(fn, args, kwargs)
            finally:
                torch.cuda.nvtx.range_pop()
        try:
            with set_current_context(target):
                out = self._call_in_context(fn, args, kwargs)
            if debug_utils.active_checks():
                debug_utils.check_outputs(out, where=f"{self.path()} [{type(self).__name__}.{fn.__name__}]")
            return out
        except Exception as e:  # pylint: disable=broad-except
            # One line per module on the way out: the traceback then names WHICH layer failed.
            traceback_util.add_module_note(e, path=self.path(), cls=type(self).__name__, method=fn.__name__)
            raise

    wrapped.__wrapped_module_method__ = True
    return wrapped


# --------------------------------------------------------------------------------------
# Module.
# --------------------------------------------------------------------------------------


class Module(Configurable):
    """A named node in a tree of modules."""

    @config_class
    class Config(Configurable.Config):
        name: Required[str] = REQUIRED
        # Verbosity for vlog(); messages at level <= vlog are emitted.
        vlog: Optional[int] = None

    # Methods that are never wrapped even though they are public.
    _NEVER_WRAP = frozenset(
        {
            "default_config",
            "path",
            "vlog_is_on",
            "vlog",
            "vprint",
            "get_invocation_context",
            "add_summary",
            "add_state_update",
            "add_module_output",
            "get_module_outputs",
            "get_shared_module",
        }
    )

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        for name, attr in list(cls.__dict__.items()):
            if name.startswith("_") or name in Module._NEVER_WRAP:
                continue
            if not callable(attr) or isinstance(attr, (type, staticmethod, classmethod, property)):
                continue
            if getattr(attr, "__nowrap__", False) or getattr(
                attr, "__wrapped_module_method__", False
            ):
                continue
            setattr(cls, name, _wrap_method(attr))

    def __init__(self, cfg: "Module.Config", *, parent: Optional["Module"] = None):
        super().__init__(cfg)
        name = cfg.name
        if not isinstance(name, str) or not _NAME_RE.fullmatch(name):
            raise ValueError(f'Invalid module name "{name}"')
        self._name = name
        self._parent = parent
        self._children: dict[str, Module] = {}
        self._shared: dict[str, Module] = {}
        self._vlog_level = cfg.vlog

    # ------------------------------------------------------------------ tree
    @property
    def name(self) -> str:
        return self._name

    @property
    def parent(self) -> Optional["Module"]:
        return self._parent

    @property
    def children(self) -> dict[str, "Module"]:
        return dict(self._children)

    def path(self) -> str:
        if self._parent is None:
            return self._name
        return f"{self._parent.path()}.{self._name}"

    def __getattr__(self, name: str) -> Any:
        # Only reached when normal lookup fails: resolve children by name.
        kids = self.__dict__.get("_children")
        if kids is not None and name in kids:
            return kids[name]
        raise AttributeError(f"{type(self).__name__} has no attribute or child {name!r}")

    def _add_child(self, name: str, child_config: "Module.Config", **kwargs) -> "Module":
        """Instantiates ``child_config`` as a child called ``name``."""
        if not _NAME_RE.fullmatch(name):
            raise ValueError(f'Invalid child name "{name}"')
        if name in self._children:
            raise ValueError(f'{self.path()} already has a child named "{name}"')
        if name in self.__dict__ or hasattr(type(self), name):
            raise ValueError(f'Child name "{name}" shadows an attribute of {type(self).__name__}')
        child = child_config.clone(name=name).instantiate(parent=self, **kwargs)
        self._children[name] = child
        return child

    def _share_with_descendants(self, module: "Module", *, shared_module_name: str) -> None:
        """Makes ``module`` reachable from any descendant via get_shared_module()."""
        self._shared[shared_module_name] = module

    def get_shared_module(self, shared_module_name: str) -> "Module":
        node: Optional[Module] = self
        while node is not None:
            if shared_module_name in node._shared:
                return node._shared[shared_module_name]
            node = node._parent
        raise KeyError(f"No ancestor of {self.path()} shares a module {shared_module_name!r}")

    # ------------------------------------------------------------------ context plumbing
    def _call_in_context(self, fn: Callable, args: tuple, kwargs: dict) -> Any:
        """Hook around every wrapped call made from another module (after this module's
        context has been entered).  BaseLayer overrides it to apply rematerialisation."""
        return fn(self, *args, **kwargs)

    def _resolve_context(self, cur: InvocationContext) -> InvocationContext:
        """Finds (or derives) the context in which a method of ``self`` must run when the
        innermost active context is ``cur``."""
        # Fast path: direct child.
        if self._parent is cur.module and cur.module._children.get(self._name) is self:
            return cur.add_child(self._name)
        # Descendant: derive the chain of child contexts.
        chain: list[Module] = []
        node: Optional[Module] = self
        while node is not None and node is not cur.module:
            chain.append(node)
            node = node._parent
        if node is cur.module:
            ctx = cur
            for m in reversed(chain):
                ctx = ctx.add_child(m._name)
            return ctx
        # Ancestor or shared module: find the first context up the stack that can reach it.
        up: Optional[InvocationContext] = cur.parent
        while up is not None:
            if up.module is self:
                return up
            chain = []
            node = self
            while node is not None and node is not up.module:
                chain.append(node)
                node = node._parent
            if node is up.module:
                ctx = up
                for m in reversed(chain):
                    ctx = ctx.add_child(m._name)
                return ctx
            up = up.parent
        raise ValueError(
            f"Module {self.path()} is not reachable from invocation context {cur.path()}"
        )

    def get_invocation_context(self) -> InvocationContext:
        ctx = current_context()
        if ctx is None:
            raise RuntimeError(f"{self.path()}: no invocation context is active")
        if ctx.module is not self:
            raise RuntimeError(
                f"{self.path()}: active context belongs to {ctx.module.path()}"
            )
        return ctx

    @property
    def is_training(self) -> bool:
        return self.get_invocation_context().is_training

    @property
    def prng_key(self) -> torch.Tensor:
        key = self.get_invocation_context().prng_key
        if key is None:
            raise ValueError(f"{self.path()}: this call was made without a prng_key")
        return key

    @property
    def state(self) -> Any:
        return self.get_invocation_context().state

    def add_summary(self, name: str, value: Any) -> None:
        self.get_invocation_context().add_summary(name, value)

    def add_state_update(self, name: str, value: Any) -> None:
        self.get_invocation_context().add_state_update(name, value)

    def add_module_output(self, name: str, value: Any) -> None:
        self.get_invocation_context().add_module_output(name, value)

    def get_module_outputs(self) -> dict:
        return self.get_invocation_context().get_module_outputs()

    # ------------------------------------------------------------------ logging
    def vlog_is_on(self, level: int) -> bool:
        return self._vlog_level is not None and level <= self._vlog_level

    def vlog(self, level: int, msg: str, *args) -> None:
        if self.vlog_is_on(level):
            import logging

            logging.getLogger("axlearn_b200").info("@%s " + msg, self.path(), *args)

    def vprint(self, level: int, msg: str, *args, **kwargs) -> None:
        if self.vlog_is_on(level):
            print(f"@{self.path()} " + msg.format(*args, **kwargs))

    def __call__(self, *args, **kwargs) -> Any:
        """Shorthand for ``self.forward(...)``."""
        return self.forward(*args, **kwargs)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.path()})"


# --------------------------------------------------------------------------------------
# functional() and scan_in_context().
# --------------------------------------------------------------------------------------


def functional(
    module: Module,
    prng_key: Optional[torch.Tensor],
    state: Any,
    inputs: Union[Sequence[Any], dict[str, Any]],
    *,
    method: str = "forward",
    is_training: bool,
    drop_output_collections: Sequence[str] = ("module_outputs",),
) -> tuple[Any, OutputCollection]:
    """Invokes ``module.method(*inputs)`` (or ``**inputs``) in a fresh root context.

    Returns ``(method_outputs, output_collection)``.  Collections listed in
    ``drop_output_collections`` are emptied before returning (module outputs can be large
    activations that callers rarely want).
    """
    ctx = InvocationContext(
        name="root",
        parent=None,
        module=module,
        state=state,
        is_training=is_training,
        prng_key=prng_key,
        output_collection=new_output_collection(),
    )
    fn = getattr(module, method)
    with set_current_context(ctx, require_parent=False):
        if isinstance(inputs, dict):
            out = fn(**inputs)
        else:
            out = fn(*inputs)
    oc = ctx.output_collection
    for name in drop_output_collections:
        getattr(oc, name).clear()
    return out, oc


def scan_in_context(
    fn: Callable[[Any, Any], tuple[Any, Any]],
    *,
    carry: Any,
    xs: Any,
    num_iters: Optional[int] = None,
    drop_output: Optional[Callable[[str], bool]] = None,
    child_name_prefix: str = "iter",
    stack_outputs: bool = True,
) -> tuple[Any, Any]:
    """Runs ``carry, y_i = fn(carry, x_i)`` for each leading-dim slice ``x_i`` of ``xs``.

    Each iteration's summaries / module outputs are stored under ``{prefix}{i}`` of the
    current module's output collection.  ``ys`` are stacked on a new leading dim (or
    returned as a list with ``stack_outputs=False``).
    """
    from axlearn_b200.common.utils import tree_map  # Local import: utils imports module.

    ctx = current_context()
    if ctx is None:
        raise RuntimeError("scan_in_context() needs an invocation context")
    leaves = _tree_leaves(xs)
    if num_iters is None:
        if not leaves:
            raise ValueError("num_iters is required when xs has no tensors")
        num_iters = leaves[0].shape[0]
    ys: list[Any] = []
    per_iter: list[OutputCollection] = []
    for i in range(num_iters):
        x_i = tree_map(lambda t, i=i: t[i], xs)
        iter_ctx = dataclasses.replace(
            ctx,
            output_collection=new_output_collection(),
            prng_key=None if ctx.prng_key is None else prng.fold_in(ctx.prng_key, i),
        )
        # The iteration context stands in for ``ctx`` (same module), so children resolve.
        with set_current_context(iter_ctx, require_parent=False):
            carry, y_i = fn(carry, x_i)
        ys.append(y_i)
        oc = iter_ctx.output_collection
        if drop_output is not None:
            for coll in (oc.summaries, oc.module_outputs):
                _prune_paths(coll, drop_output)
        per_iter.append(oc)
    propagate_repeated_output_collections(
        per_iter, child_name_prefix=child_name_prefix, target=ctx.output_collection
    )
    if stack_outputs and ys and _tree_leaves(ys[0]):
        ys = tree_map(lambda *ts: torch.stack(ts, dim=0), *ys)
    return carry, ys


def _tree_leaves(tree: Any) -> list[torch.Tensor]:
    out: list[torch.Tensor] = []
    if isinstance(tree, torch.Tensor):
        out.append(tree)
    elif isinstance(tree, dict):
        for k in tree:
            out.extend(_tree_leaves(tree[k]))
    elif isinstance(tree, (list, tuple)):
        for v in tree:
            out.extend(_tree_leaves(v))
    return out


def _prune_paths(tree: dict, drop: Callable[[str], bool], prefix: str = "") -> None:
    for k in list(tree.keys()):
        path = f"{prefix}/{k}" if prefix else k
        if isinstance(tree[k], dict):
            _prune_paths(tree[k], drop, path)
        elif drop(path):
            del tree[k]
