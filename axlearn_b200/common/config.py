"""Composable, partially-specified configuration objects.

A config is a typed bag of fields, declared with ``@config_class`` on a subclass of
``ConfigBase``.  Configs are values: assignment deep-copies mutable inputs, ``clone()``
duplicates the whole tree, and ``Configurable`` instances keep a private frozen copy.
``InstantiableConfig.instantiate()`` turns a fully-specified config into the object it
describes.  This file deliberately imports no tensor library so that configs can be built,
printed and diffed on any host.

Behavioural parity targets in the reference (axlearn/common/config.py): ``REQUIRED`` /
``Required`` (:145-258), validators (:298-410), ``ConfigBase`` (:488-846), ``config_class``
(:850), ``InstantiableConfig`` (:887), ``Configurable`` (:923), ``config_for_function``
(:1082), ``config_for_class`` (:1144), ``maybe_set_config`` (:1182), ``ConfigModifier``
(:1190), ``get_named_trainer_config`` (:1213).

The implementation here is metaclass-free and has no third-party dependency: field tables
are plain dicts attached to each decorated class.
"""

from __future__ import annotations

import copy
import dataclasses
import difflib
import enum
import importlib
import inspect
import re
import types
from collections import defaultdict
from collections.abc import Collection, Iterable, Sequence
from typing import Any, Callable, Generic, Optional, TypeVar, Union

__all__ = [
    "REQUIRED",
    "Required",
    "RequiredFieldValue",
    "ConfigBase",
    "ConfigOr",
    "Configurable",
    "ConfigModifier",
    "FunctionConfigBase",
    "ClassConfigBase",
    "InstantiableConfig",
    "InvalidConfigClassError",
    "InvalidConfigNameError",
    "InvalidConfigValueError",
    "MissingConfigClassDecoratorError",
    "NonConfigFieldError",
    "RequiredFieldMissingError",
    "UnknownFieldError",
    "TrainerConfigFn",
    "config_class",
    "config_for_class",
    "config_for_function",
    "get_named_trainer_config",
    "maybe_instantiate",
    "maybe_set_config",
    "register_validator",
    "similar_names",
    "validate_config_field_name",
    "validate_config_field_value",
]

T = TypeVar("T")


# --------------------------------------------------------------------------------------
# Errors.
# --------------------------------------------------------------------------------------


class InvalidConfigClassError(TypeError):
    """A class decorated with @config_class is malformed."""


class MissingConfigClassDecoratorError(TypeError):
    """A ConfigBase subclass was used without @config_class."""


class NonConfigFieldError(InvalidConfigClassError):
    """A config class defines a public attribute that is not an annotated field."""


class InvalidConfigNameError(ValueError):
    """A field name violates the naming rule."""


class InvalidConfigValueError(TypeError):
    """A field value is of a type that configs may not hold."""


class UnknownFieldError(AttributeError):
    """Access to a field that the config does not declare."""


class RequiredFieldMissingError(ValueError):
    """instantiate() was called while a REQUIRED field is unset."""


# --------------------------------------------------------------------------------------
# REQUIRED sentinel.
# --------------------------------------------------------------------------------------


class RequiredFieldValue:
    """Singleton marker for fields the user must set before instantiate()."""

    _instance: Optional["RequiredFieldValue"] = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
        return cls._instance

    def __bool__(self):
        return False

    def __repr__(self):
        return "REQUIRED"

    def __deepcopy__(self, memo):
        return self

    def __copy__(self):
        return self

    def __reduce__(self):
        return (RequiredFieldValue, ())


REQUIRED = RequiredFieldValue()
Required = Union[T, RequiredFieldValue]


# --------------------------------------------------------------------------------------
# Validation.
# --------------------------------------------------------------------------------------

_FIELD_NAME_RE = re.compile(r"^[a-z][a-z0-9_]*$")
_RESERVED_NAMES: set[str] = set()  # Filled in after ConfigBase is defined.


def validate_config_field_name(name: str) -> None:
    """Field names are lower snake case and must not shadow ConfigBase attributes."""
    if not isinstance(name, str) or not _FIELD_NAME_RE.fullmatch(name):
        raise InvalidConfigNameError(f'Invalid config field name "{name}"')
    if name in _RESERVED_NAMES:
        raise InvalidConfigNameError(f'"{name}" is a reserved config attribute name')


# An ordered registry of (match_fn, validate_fn). The first matching entry decides.
_validators: list[tuple[Callable[[Any], bool], Callable[[Any], None]]] = []


def register_validator(
    *, match_fn: Callable[[Any], bool], validate_fn: Callable[[Any], None]
) -> None:
    """Registers a validator for values for which ``match_fn(value)`` is true."""
    _validators.append((match_fn, validate_fn))


def _is_named_tuple(v: Any) -> bool:
    return isinstance(v, tuple) and hasattr(type(v), "_fields")


def validate_config_field_value(value: Any) -> None:
    """Raises InvalidConfigValueError unless ``value`` may be stored in a config."""
    for match_fn, validate_fn in _validators:
        if match_fn(value):
            validate_fn(value)
            return
    raise InvalidConfigValueError(
        f'Config values of type "{type(value)}" are not supported: {value!r}'
    )


def _noop(_):
    return None


def _validate_seq(v):
    for x in v:
        validate_config_field_value(x)


def _validate_dict(v):
    for k, x in v.items():
        if not isinstance(k, (str, int, enum.Enum, tuple)):
            raise InvalidConfigValueError(f'Dict key "{k!r}" must be str/int/enum/tuple')
        validate_config_field_value(x)


def _validate_dataclass(v):
    for f in dataclasses.fields(v):
        validate_config_field_value(getattr(v, f.name))


register_validator(
    match_fn=lambda v: v is None
    or v is REQUIRED
    or isinstance(v, (bool, int, float, complex, str, bytes, enum.Enum, type, slice))
    or isinstance(
        v,
        (
            types.FunctionType,
            types.BuiltinFunctionType,
            types.MethodType,
            types.ModuleType,
            re.Pattern,
        ),
    ),
    validate_fn=_noop,
)
register_validator(match_fn=lambda v: isinstance(v, ConfigBase), validate_fn=_noop)
register_validator(match_fn=lambda v: isinstance(v, (defaultdict, dict)), validate_fn=_validate_dict)
register_validator(
    match_fn=lambda v: isinstance(v, (list, tuple, set, frozenset)), validate_fn=_validate_seq
)
register_validator(
    match_fn=lambda v: dataclasses.is_dataclass(v) and not isinstance(v, type),
    validate_fn=_validate_dataclass,
)
# Opaque leaves that are known to be safe values: dtypes, devices, numpy scalars, callables
# implementing __call__ (e.g. functools.partial) are accepted by duck-typing below.
register_validator(
    match_fn=lambda v: type(v).__module__.split(".")[0] in ("torch", "numpy", "functools"),
    validate_fn=_noop,
)
register_validator(match_fn=lambda v: hasattr(v, "__config_value__"), validate_fn=_noop)


def similar_names(name: str, candidates: Iterable[str]) -> list[str]:
    """Candidate names close to ``name`` (closest first), for "did you mean" hints."""
    scored = []
    for cand in candidates:
        ratio = difflib.SequenceMatcher(None, name, cand).ratio()
        if ratio >= 0.75 or name in cand or cand in name:
            scored.append((-ratio, cand))
    return [c for _, c in sorted(scored)]


# --------------------------------------------------------------------------------------
# Field table.
# --------------------------------------------------------------------------------------


@dataclasses.dataclass(frozen=True)
class _Field:
    name: str
    type: Any
    default: Any
    mutable: bool = True  # False => value is shared, not copied (e.g. ``klass``/``fn``).


_FIELDS_ATTR = "__config_fields__"
_DECORATED_ATTR = "__config_class_of__"


def _fields_of(cls: type) -> dict[str, _Field]:
    if cls.__dict__.get(_DECORATED_ATTR) is not cls:
        raise MissingConfigClassDecoratorError(
            f"{cls.__qualname__} must be decorated with @config_class"
        )
    return cls.__dict__[_FIELDS_ATTR]


def _copy_value(v: Any) -> Any:
    """Copies containers/configs so that configs never alias caller-owned mutable state."""
    if isinstance(v, ConfigBase):
        return v.clone()
    if isinstance(v, defaultdict):
        out = defaultdict(v.default_factory)
        for k, x in v.items():
            out[k] = _copy_value(x)
        return out
    if isinstance(v, dict):
        return type(v)((k, _copy_value(x)) for k, x in v.items())
    if _is_named_tuple(v):
        return type(v)(*[_copy_value(x) for x in v])
    if isinstance(v, (list, tuple, set, frozenset)):
        return type(v)(_copy_value(x) for x in v)
    if dataclasses.is_dataclass(v) and not isinstance(v, type):
        return copy.deepcopy(v)
    return v


def config_class(cls: type[T]) -> type[T]:
    """Class decorator that turns annotated attributes into config fields.

    Fields are the union of the annotated attributes along the MRO; a subclass may
    re-declare a field to change its default.  Public non-annotated, non-callable
    attributes are rejected so that a forgotten annotation is caught early.
    """
    if not (isinstance(cls, type) and issubclass(cls, ConfigBase)):
        raise InvalidConfigClassError(f"@config_class target {cls} must subclass ConfigBase")
    fields: dict[str, _Field] = {}
    for base in reversed(cls.__mro__[1:]):
        base_fields = base.__dict__.get(_FIELDS_ATTR)
        if base_fields:
            fields.update(base_fields)
    annotations = cls.__dict__.get("__annotations__", {})
    if isinstance(annotations, dict) is False:  # pragma: no cover
        annotations = dict(annotations)
    for name, tp in annotations.items():
        if name.startswith("__"):
            continue
        validate_config_field_name(name)
        default = cls.__dict__.get(name, REQUIRED)
        if isinstance(default, (classmethod, staticmethod, property)):
            raise InvalidConfigClassError(
                f"{cls.__qualname__}.{name}: field default may not be a method/property"
            )
        validate_config_field_value(default)
        fields[name] = _Field(name=name, type=tp, default=default)
    for name, value in cls.__dict__.items():
        if name.startswith("_") or name in annotations:
            continue
        if callable(value) or isinstance(value, (classmethod, staticmethod, property)):
            continue
        raise NonConfigFieldError(
            f"{cls.__qualname__}.{name} is a public attribute without a type annotation"
        )
    # Defaults live in the field table, not as class attributes, so that __getattr__ on an
    # instance is the single source of truth.
    for name in annotations:
        if name in cls.__dict__ and not name.startswith("__"):
            delattr(cls, name)
    setattr(cls, _FIELDS_ATTR, fields)
    setattr(cls, _DECORATED_ATTR, cls)
    return cls


class ConfigBase:
    """Base class of all configs. Subclasses must be decorated with @config_class."""

    __slots__ = ("_values",)

    def __init__(self, **kwargs):
        fields = _fields_of(type(self))
        object.__setattr__(self, "_values", {})
        for name, f in fields.items():
            self._values[name] = _copy_value(f.default) if f.mutable else f.default
        for k, v in kwargs.items():
            setattr(self, k, v)

    # ------------------------------------------------------------------ attribute access
    def __getattr__(self, name: str) -> Any:
        if name == "_values":
            raise AttributeError(name)
        try:
            return self._values[name]
        except KeyError:
            raise self._unknown(name) from None

    def __setattr__(self, name: str, value: Any) -> None:
        fields = _fields_of(type(self))
        f = fields.get(name)
        if f is None:
            raise self._unknown(name)
        validate_config_field_value(value)
        self._values[name] = _copy_value(value) if f.mutable else value

    def __delattr__(self, name: str) -> None:
        raise AttributeError(f"Config fields cannot be deleted: {name}")

    def _unknown(self, name: str) -> UnknownFieldError:
        hint = similar_names(name, self.keys())
        msg = f"{type(self).__qualname__} has no field {name!r}"
        if hint:
            msg += f"; did you mean: [{', '.join(hint)}]"
        return UnknownFieldError(msg)

    def __contains__(self, name: str) -> bool:
        return name in self._values

    def __len__(self) -> int:
        return len(self._values)

    def keys(self) -> list[str]:
        return list(self._values.keys())

    def items(self) -> list[tuple[str, Any]]:
        return list(self._values.items())

    def __eq__(self, other: Any) -> bool:
        return type(other) is type(self) and self._values == other._values

    def __ne__(self, other):
        return not self == other

    __hash__ = None  # Configs are mutable values.

    def __repr__(self) -> str:
        return f"{type(self).__qualname__}({', '.join(f'{k}={v!r}' for k, v in self.items())})"

    def __str__(self) -> str:
        return self.debug_string()

    def __deepcopy__(self, memo):
        return self.clone()

    def __getstate__(self):
        return dict(self._values)

    def __setstate__(self, state):
        object.__setattr__(self, "_values", dict(state))

    def __reduce__(self):
        return (_rebuild_config, (type(self), dict(self._values)))

    # ------------------------------------------------------------------ mutation helpers
    def set(self, **kwargs):
        """Sets several fields; returns self to allow chaining."""
        for k, v in kwargs.items():
            setattr(self, k, v)
        return self

    def clone(self, **kwargs):
        """Deep copy with optional overrides; the original is left untouched."""
        new = object.__new__(type(self))
        fields = _fields_of(type(self))
        object.__setattr__(
            new,
            "_values",
            {
                k: (_copy_value(v) if fields[k].mutable else v)
                for k, v in self._values.items()
            },
        )
        return new.set(**kwargs)

    def get_recursively(self, path: Sequence[str]) -> Any:
        cur = self
        for key in path:
            cur = getattr(cur, key)
        return cur

    def set_recursively(self, path: Sequence[str], *, value: Any) -> None:
        if not path:
            raise ValueError("Path is empty.")
        setattr(self.get_recursively(path[:-1]), path[-1], value)

    # ------------------------------------------------------------------ traversal
    def visit(
        self,
        visit_fn: Callable[[str, Any], None],
        *,
        enter_fn: Optional[Callable[[str, Any, Optional[list]], Optional[list]]] = None,
    ) -> None:
        """Depth-first walk over leaves.

        Paths use ``a.b`` for sub-configs, ``a[0]`` for sequence items and ``a['k']`` for
        dict / dataclass members.  ``enter_fn(key, val, default_children)`` may return a
        replacement list of ``(key, value)`` children (``[]`` prunes; ``None`` makes the
        node a leaf).
        """

        def children(key: str, val: Any) -> Optional[list]:
            if isinstance(val, ConfigBase):
                pre = f"{key}." if key else ""
                return [(f"{pre}{k}", v) for k, v in val.items()]
            if isinstance(val, dict):
                return [(f"{key}[{k!r}]", v) for k, v in val.items()]
            if _is_named_tuple(val):
                return [(f"{key}[{f!r}]", getattr(val, f)) for f in val._fields]
            if isinstance(val, (list, tuple)):
                return [(f"{key}[{i}]", v) for i, v in enumerate(val)]
            if dataclasses.is_dataclass(val) and not isinstance(val, type):
                return [
                    (f"{key}[{f.name!r}]", getattr(val, f.name)) for f in dataclasses.fields(val)
                ]
            return None

        def walk(key: str, val: Any) -> None:
            kids = children(key, val)
            if enter_fn is not None:
                kids = enter_fn(key, val, kids)
            if kids is None:
                visit_fn(key, val)
                return
            for k, v in kids:
                walk(k, v)

        walk("", self)

    def to_flat_dict(self, *, omit_default_values: Collection[Any]) -> dict[str, Any]:
        """``{path: leaf}``; a leaf still at its default is dropped when that default is
        one of ``omit_default_values`` (compared by identity or equality of simple values)."""
        out: dict[str, Any] = {}
        fields = _fields_of(type(self))

        def omitted(default: Any, val: Any) -> bool:
            return val is default and any(default is o for o in omit_default_values)

        def enter(key: str, val: Any, default_children: Optional[list]) -> Optional[list]:
            if key and isinstance(val, ConfigBase):
                sub = val.to_flat_dict(omit_default_values=omit_default_values)
                out.update({f"{key}.{k}": v for k, v in sub.items()})
                return []
            if dataclasses.is_dataclass(val) and not isinstance(val, type):
                defaults = {f"{key}[{f.name!r}]": f.default for f in dataclasses.fields(val)}
                return [
                    (k, v) for k, v in default_children if not omitted(defaults.get(k), v)
                ]
            return default_children

        def leaf(key: str, val: Any) -> None:
            f = fields.get(key)
            if f is not None and omitted(f.default, val):
                return
            out[key] = val

        self.visit(leaf, enter_fn=enter)
        return out

    def debug_string(
        self,
        *,
        kv_separator: str = ": ",
        field_separator: str = "\n",
        omit_default_values: Collection[Any] = (None, REQUIRED),
    ) -> str:
        """One ``path: repr(value)`` entry per leaf; classes and functions print as
        ``module.name`` so that the string is stable across processes."""

        def fmt(v: Any) -> str:
            if isinstance(v, (type, types.FunctionType)):
                return repr(f"{v.__module__}.{v.__name__}")
            return repr(v)

        flat = self.to_flat_dict(omit_default_values=omit_default_values)
        return field_separator.join(f"{k}{kv_separator}{fmt(v)}" for k, v in flat.items())

    def to_dict(self) -> dict[str, Any]:
        """Nested plain-dict view (sub-configs become dicts, types become dotted names)."""

        def conv(v: Any) -> Any:
            if isinstance(v, ConfigBase):
                return v.to_dict()
            if isinstance(v, dict):
                return {k: conv(x) for k, x in v.items()}
            if _is_named_tuple(v):
                return {f: conv(getattr(v, f)) for f in v._fields}
            if isinstance(v, (list, tuple)):
                return [conv(x) for x in v]
            if dataclasses.is_dataclass(v) and not isinstance(v, type):
                return conv(dataclasses.asdict(v))
            if isinstance(v, (type, types.FunctionType)):
                return f"{v.__module__}.{v.__qualname__}"
            if isinstance(v, enum.Enum):
                return str(v)
            return v

        return {k: conv(v) for k, v in self.items()}


def _rebuild_config(cls, values):
    new = object.__new__(cls)
    object.__setattr__(new, "_values", values)
    return new


_RESERVED_NAMES.update(n for n in dir(ConfigBase) if not n.startswith("_"))


# --------------------------------------------------------------------------------------
# Instantiable configs.
# --------------------------------------------------------------------------------------


def _check_required(cfg: ConfigBase) -> None:
    missing: list[str] = []

    def visit(key, val):
        if val is REQUIRED:
            missing.append(key)

    def enter(key, val, kids):
        # Nested instantiable configs are checked when *they* are instantiated.
        if key and isinstance(val, InstantiableConfig):
            return []
        return kids

    cfg.visit(visit, enter_fn=enter)
    if missing:
        raise RequiredFieldMissingError(
            f"Missing value for required field(s) {missing} when instantiating "
            f"{type(cfg).__qualname__}:\n{cfg.debug_string(omit_default_values=())}"
        )


@config_class
class InstantiableConfig(ConfigBase, Generic[T]):
    """A config that knows how to build the object it describes."""

    def instantiate(self, **kwargs) -> T:
        raise NotImplementedError(type(self))


ConfigOr = Union[T, InstantiableConfig]


def maybe_instantiate(x: Any) -> Any:
    """Instantiates ``x`` if it is an InstantiableConfig, else returns it unchanged."""
    if isinstance(x, InstantiableConfig):
        return x.instantiate()
    return x


class Configurable:
    """Base class of objects built from a ``Config``.

    Subclasses declare ``@config_class class Config(Base.Config)`` and are created with
    ``Cls.default_config().set(...).instantiate(...)``.
    """

    @config_class
    class Config(InstantiableConfig):
        klass: type = REQUIRED

        def instantiate(self, **kwargs):
            _check_required(self)
            return self.klass(self, **kwargs)

    @classmethod
    def default_config(cls) -> "Configurable.Config":
        cfg_cls = cls.Config
        _fields_of(cfg_cls)  # Raises if the decorator is missing.
        cfg = cfg_cls()
        cfg._values["klass"] = cls
        return cfg

    def __init__(self, cfg: "Configurable.Config"):
        self._config = cfg.clone()

    @property
    def config(self) -> "Configurable.Config":
        """A copy of the config; mutating it does not affect this object."""
        return self._config.clone()

    def __repr__(self):
        return f"{type(self)}({self._config!r})"


# ``klass`` refers to a class object and must never be copied.
Configurable.Config.__config_fields__["klass"] = dataclasses.replace(
    Configurable.Config.__config_fields__["klass"], mutable=False
)


@config_class
class FunctionConfigBase(InstantiableConfig):
    """Config synthesised from a function signature; instantiate() calls the function."""

    fn: Any = REQUIRED

    def instantiate(self, **kwargs):
        _check_required(self)
        args, call_kwargs = _bind(self, inspect.signature(self.fn), skip=("fn",))
        call_kwargs.update(kwargs)
        return self.fn(*args, **call_kwargs)


@config_class
class ClassConfigBase(InstantiableConfig):
    """Config synthesised from ``cls.__init__``; instantiate() constructs the class."""

    klass: type = REQUIRED

    def instantiate(self, **kwargs):
        _check_required(self)
        sig = inspect.signature(self.klass.__init__)
        params = list(sig.parameters.values())[1:]  # Drop self.
        args, call_kwargs = _bind(self, sig.replace(parameters=params), skip=("klass",))
        call_kwargs.update(kwargs)
        return self.klass(*args, **call_kwargs)


def _bind(cfg: ConfigBase, sig: inspect.Signature, *, skip: Sequence[str]):
    """Maps config fields back onto positional / keyword / variadic parameters."""
    args: list[Any] = []
    kwargs: dict[str, Any] = {}
    values = {k: maybe_instantiate_nested(v) for k, v in cfg.items() if k not in skip}
    params = list(sig.parameters.values())
    # Once *args is non-empty, everything declared before it has to travel positionally.
    has_varargs = any(
        p.kind is inspect.Parameter.VAR_POSITIONAL and values.get(p.name) for p in params
    )
    for p in params:
        if p.name not in values:
            continue
        v = values[p.name]
        if p.kind is inspect.Parameter.VAR_POSITIONAL:
            args.extend(v)
        elif p.kind is inspect.Parameter.VAR_KEYWORD:
            kwargs.update(v)
        elif p.kind is inspect.Parameter.POSITIONAL_ONLY or (
            has_varargs and p.kind is inspect.Parameter.POSITIONAL_OR_KEYWORD
        ):
            args.append(v)
        else:
            kwargs[p.name] = v
    return args, kwargs


def maybe_instantiate_nested(v: Any) -> Any:
    """Function/class configs pass their values through unchanged; nested configs are the
    callee's business (matching the reference, which hands sub-configs to the callee)."""
    return v


def _synthesise(
    base: type, target: Callable, sig: inspect.Signature, *, handle_name: str, qualname: str
) -> type:
    annotations: dict[str, Any] = {}
    namespace: dict[str, Any] = {}
    for p in sig.parameters.values():
        if p.name in (handle_name,):
            raise InvalidConfigClassError(
                f'Parameter name "{p.name}" of {target} collides with the config handle field'
            )
        validate_config_field_name(p.name)
        annotations[p.name] = p.annotation if p.annotation is not inspect.Parameter.empty else Any
        if p.kind is inspect.Parameter.VAR_POSITIONAL:
            default = []
        elif p.kind is inspect.Parameter.VAR_KEYWORD:
            default = {}
        elif p.default is inspect.Parameter.empty:
            default = REQUIRED
        else:
            default = p.default
        namespace[p.name] = default
    namespace["__annotations__"] = annotations
    namespace["__qualname__"] = qualname
    namespace["__module__"] = getattr(target, "__module__", __name__)
    new_cls = config_class(type(f"config_for({qualname})", (base,), namespace))
    new_cls.__config_fields__[handle_name] = dataclasses.replace(
        new_cls.__config_fields__[handle_name], mutable=False
    )
    return new_cls


_fn_cfg_cache: dict[Any, type] = {}


def config_for_function(fn: Callable[..., T]) -> FunctionConfigBase:
    """Returns a config whose fields mirror ``fn``'s parameters.

    Parameters without defaults become REQUIRED; ``*args`` defaults to ``[]`` and
    ``**kwargs`` to ``{}``.
    """
    if not callable(fn) or isinstance(fn, type):
        raise InvalidConfigValueError(f"config_for_function expects a function, got {fn!r}")
    try:
        cfg_cls = _fn_cfg_cache.get(fn)
    except TypeError:
        cfg_cls = None
    if cfg_cls is None:
        name = getattr(fn, "__qualname__", repr(fn))
        cfg_cls = _synthesise(
            FunctionConfigBase, fn, inspect.signature(fn), handle_name="fn", qualname=name
        )
        try:
            _fn_cfg_cache[fn] = cfg_cls
        except TypeError:
            pass
    cfg = cfg_cls()
    cfg._values["fn"] = fn
    return cfg


def config_for_class(cls: type[T]) -> ClassConfigBase:
    """Returns a config whose fields mirror ``cls.__init__``'s parameters."""
    if not isinstance(cls, type):
        raise InvalidConfigValueError(f"config_for_class expects a class, got {cls!r}")
    cfg_cls = _fn_cfg_cache.get(cls)
    if cfg_cls is None:
        init_sig = inspect.signature(cls.__init__)
        params = list(init_sig.parameters.values())[1:]
        if cls.__init__ is object.__init__:
            params = []
        cfg_cls = _synthesise(
            ClassConfigBase,
            cls,
            init_sig.replace(parameters=params),
            handle_name="klass",
            qualname=cls.__qualname__,
        )
        _fn_cfg_cache[cls] = cfg_cls
    cfg = cfg_cls()
    cfg._values["klass"] = cls
    return cfg


def maybe_set_config(cfg: ConfigBase, **kwargs) -> ConfigBase:
    """Sets only those fields that ``cfg`` actually declares."""
    for k, v in kwargs.items():
        if k in cfg:
            setattr(cfg, k, v)
    return cfg


class ConfigModifier(Configurable):
    """A callable ``cfg -> cfg`` built from a config; used by mesh rules to rewrite trainer
    configs for a particular hardware target."""

    def __call__(self, cfg: InstantiableConfig) -> InstantiableConfig:
        raise NotImplementedError(type(self))


TrainerConfigFn = Callable[[], InstantiableConfig]


def get_named_trainer_config(
    config_name: str, *, config_module: str, root_module: Optional[str] = None
) -> TrainerConfigFn:
    """Looks up ``config_name`` in ``config_module.named_trainer_configs()``.

    ``config_module`` is tried as given and, failing that, as
    ``{root_module}.experiments.{config_module}``.
    """
    candidates = [config_module]
    if root_module:
        candidates.append(f"{root_module}.experiments.{config_module}")
    module = None
    err: Optional[Exception] = None
    for name in candidates:
        try:
            module = importlib.import_module(name)
            break
        except ImportError as e:
            err = e
    if module is None:
        raise ImportError(f"Cannot import any of {candidates}") from err
    configs = module.named_trainer_configs()
    if config_name not in configs:
        hint = similar_names(config_name, configs.keys())
        raise KeyError(
            f"Unknown trainer config {config_name!r} in {module.__name__}"
            + (f"; did you mean: {hint}" if hint else "")
        )
    return configs[config_name]
