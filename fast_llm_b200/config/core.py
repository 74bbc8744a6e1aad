"""Declarative configuration system.

A config class is a plain Python class whose annotated attributes are *fields*.  Instances are built from nested
dictionaries (YAML), validated field by field (type coercion, range checks, derived defaults), then frozen.  Classes can
register under a name in the registry of a base class so a `type:` key selects the concrete class.  Only fields the
user set explicitly are serialised by default, so a saved config round-trips without pinning today's defaults.

Behavioural parity with `fast_llm/config.py` (Field `:116`, config_class `:231`, validate `:362-591`, to_dict `:604`,
from_dict `:725-790`, registries `:900-933`); the implementation is independent: fields are collected in
`__init_subclass__` rather than through `dataclasses`.
"""

import contextlib
import copy
import enum
import logging
import pathlib
import types
import typing

import yaml

from fast_llm_b200.utils.assertions import Assert
from fast_llm_b200.utils.misc import compare_nested

logger = logging.getLogger(__name__)

MISSING = type("MissingType", (), {"__repr__": lambda self: "MISSING", "__bool__": lambda self: False})()


class NoAutoValidate:
    """Context manager that postpones the automatic validation done by `Config.from_dict`."""

    _depth = 0

    def __enter__(self):
        NoAutoValidate._depth += 1

    def __exit__(self, *exc):
        NoAutoValidate._depth -= 1


class UpdateType(str, enum.Enum):
    override = "override"  # replace whole sub-dictionaries
    update = "update"  # merge into existing sub-dictionaries


class FieldHint(str, enum.Enum):
    core = "core"
    architecture = "architecture"
    optional = "optional"
    performance = "performance"
    stability = "stability"
    feature = "feature"
    expert = "expert"
    unknown = "unknown"
    logging = "logging"
    testing = "testing"
    derived = "derived"
    setup = "setup"
    deprecated = "deprecated"
    wip = "wip"


class FieldVerboseLevel:
    explicit = None
    core = 0
    optional = 10
    performance = 20
    debug = 50
    everything = 1000


FieldHintImportance = {
    FieldHint.core: 0,
    FieldHint.architecture: 0,
    FieldHint.optional: 10,
    FieldHint.performance: 20,
    FieldHint.stability: 20,
    FieldHint.feature: 10,
    FieldHint.expert: 30,
    FieldHint.unknown: 40,
    FieldHint.logging: 50,
    FieldHint.testing: 60,
    FieldHint.derived: 100,
    FieldHint.setup: 90,
    FieldHint.deprecated: 80,
    FieldHint.wip: 80,
}


class ValidationError(ValueError):
    pass


class Field:
    """Description of one config attribute."""

    def __init__(self, default=MISSING, *, default_factory=MISSING, desc: str | None = None, doc: str | None = None,
                 hint: FieldHint = FieldHint.unknown, valid: typing.Callable | None = None, init: bool = True):
        if default is not MISSING and default_factory is not MISSING:
            raise ValueError("cannot specify both default and default_factory")
        self.default = default
        self.default_factory = default_factory
        self.desc = desc
        self.doc = doc
        self.hint = hint
        self.valid = valid
        self.init = init
        self.name: str | None = None

    def make_default(self):
        if self.default_factory is not MISSING:
            return self.default_factory()
        if isinstance(self.default, (list, dict, set)):
            return copy.deepcopy(self.default)
        return self.default

    def clone(self, **changes) -> "Field":
        new = copy.copy(self)
        for key, value in changes.items():
            setattr(new, key, value)
        if "default" in changes:
            new.default_factory = MISSING
        if "default_factory" in changes:
            new.default = MISSING
        return new


class FieldUpdate(dict):
    """`name = FieldUpdate(default=..., hint=...)` in a subclass body changes attributes of an inherited field."""


FieldOverride = FieldUpdate


def check_field(fn: typing.Callable, *args, **kwargs) -> typing.Callable:
    def valid(x):
        fn(x, *args, **kwargs)
        return x

    return valid


def skip_valid_if_none(fn: typing.Callable, *args, **kwargs) -> typing.Callable:
    def valid(x):
        return None if x is None else fn(x, *args, **kwargs)

    return valid


def process_field(fn: typing.Callable, *args, **kwargs) -> typing.Callable:
    def valid(x):
        return fn(x, *args, **kwargs)

    return valid


def test_field(fn: typing.Callable, *args, **kwargs) -> typing.Callable:
    def valid(x):
        if not fn(x, *args, **kwargs):
            raise ValueError(f"{fn.__name__}({x}) is false")
        return x

    return valid


def _is_classvar(annotation) -> bool:
    if isinstance(annotation, str):
        return annotation.replace(" ", "").startswith(("typing.ClassVar", "ClassVar"))
    return typing.get_origin(annotation) is typing.ClassVar


def config_class(registry: bool = False, dynamic_type: "dict[type, str] | None" = None):
    """Class decorator: finalises field collection, optionally creates a registry, registers dynamic type names."""

    def wrap(cls):
        if not issubclass(cls, Config):
            raise TypeError(f"{cls.__name__} must derive from Config")
        if registry:
            cls._registry = {}
        cls._dynamic_type_names = {}
        for base, name in (dynamic_type or {}).items():
            base.register_subclass(name, cls)
            cls._dynamic_type_names[base] = name
        return cls

    return wrap


class Config:
    """Base class of all configs. See the module docstring."""

    __fields__: typing.ClassVar[dict[str, Field]] = {}
    _abstract: typing.ClassVar[bool] = False
    _registry: typing.ClassVar[dict | None] = None
    _dynamic_type_names: typing.ClassVar[dict] = {}
    _renamed_fields: typing.ClassVar[dict] = {}

    # ------------------------------------------------------------------ class construction
    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        cls._collect_fields()
        if "_abstract" not in cls.__dict__:
            cls._abstract = False

    @classmethod
    def _collect_fields(cls):
        fields: dict[str, Field] = {}
        for base in reversed(cls.__mro__[1:]):
            fields.update(base.__dict__.get("__own_fields__", {}))
        own: dict[str, Field] = {}
        for name, annotation in cls.__dict__.get("__annotations__", {}).items():
            if name.startswith("_") or _is_classvar(annotation):
                continue
            value = cls.__dict__.get(name, MISSING)
            if isinstance(value, FieldUpdate):
                continue
            field = value if isinstance(value, Field) else Field(default=value)
            field = field.clone()
            field.name = name
            own[name] = field
            if name in cls.__dict__:
                delattr(cls, name)
        for name, value in list(cls.__dict__.items()):
            if isinstance(value, FieldUpdate):
                if name not in fields and name not in own:
                    raise TypeError(f"FieldUpdate for unknown field {name} in {cls.__name__}")
                base_field = own.get(name, fields.get(name))
                own[name] = base_field.clone(**value)
                own[name].name = name
                delattr(cls, name)
        fields.update(own)
        cls.__own_fields__ = own
        cls.__fields__ = fields
        cls.__type_hints_cache__ = None

    @classmethod
    def fields(cls) -> dict[str, Field]:
        return cls.__fields__

    @classmethod
    def _type_hints(cls) -> dict[str, typing.Any]:
        if cls.__dict__.get("__type_hints_cache__") is None:
            hints = {}
            for base in reversed(cls.__mro__):
                annotations = base.__dict__.get("__annotations__", {})
                if not annotations:
                    continue
                module = __import__("sys").modules.get(base.__module__)
                namespace = dict(vars(module)) if module else {}
                namespace.setdefault(base.__name__, base)
                for name, annotation in annotations.items():
                    if isinstance(annotation, str):
                        try:
                            annotation = eval(annotation, namespace)  # noqa: S307 - annotations of our own classes
                        except Exception:
                            annotation = typing.Any
                    hints[name] = annotation
            cls.__type_hints_cache__ = hints
        return cls.__type_hints_cache__

    # ------------------------------------------------------------------ registry
    @classmethod
    def register_subclass(cls, name: str, subclass: type) -> None:
        if cls.__dict__.get("_registry") is None:
            raise TypeError(f"{cls.__name__} has no registry")
        if name in cls._registry and cls._registry[name] is not subclass:
            # Re-registration under the same name replaces the entry (module reloads in tests).
            logger.debug(f"Replacing {name} in the {cls.__name__} registry")
        cls._registry[name] = subclass

    @classmethod
    def get_subclass(cls, name: str | None) -> type:
        if name is None:
            return cls
        found = None
        for base in cls.__mro__:
            reg = base.__dict__.get("_registry")
            if reg and name in reg:
                found = reg[name]
                break
        if found is None:
            # also search registries owned by subclasses registered below this class
            stack = list(cls.__subclasses__())
            while stack and found is None:
                sub = stack.pop()
                reg = sub.__dict__.get("_registry")
                if reg and name in reg:
                    found = reg[name]
                stack.extend(sub.__subclasses__())
        if found is None:
            known = sorted({n for base in cls.__mro__ for n in (base.__dict__.get("_registry") or {})})
            raise KeyError(f"Unknown type {name!r} for base class {cls.__name__} (known: {known})")
        if not issubclass(found, cls):
            raise KeyError(f"Type {name!r} ({found.__name__}) is not a subclass of {cls.__name__}")
        return found

    @classmethod
    def _get_default_subclass(cls) -> type:
        """Concrete class used when an abstract registry base is requested without a `type`."""
        return cls

    # ------------------------------------------------------------------ instance construction
    def __init__(self, **kwargs):
        object.__setattr__(self, "_validated", False)
        object.__setattr__(self, "_explicit_fields", set())
        object.__setattr__(self, "_unknown_fields", {})
        for name, field in self.__fields__.items():
            if name in kwargs:
                value = kwargs.pop(name)
                if not field.init:
                    raise TypeError(f"Field {name} of {type(self).__name__} cannot be set explicitly")
                self._explicit_fields.add(name)
            else:
                value = field.make_default()
                if value is MISSING:
                    # nested configs always exist: default-construct them (concrete default of a registry base)
                    nested = _config_class_of(self._type_hints().get(name))
                    if nested is not None:
                        value = nested._get_default_subclass()()
            object.__setattr__(self, name, value)
        if kwargs:
            raise TypeError(f"Unknown fields for {type(self).__name__}: {sorted(kwargs)}")

    def __setattr__(self, key, value):
        if getattr(self, "_validated", False) and not key.startswith("_"):
            raise RuntimeError(f"Cannot set {key} on validated config {type(self).__name__}: configs are frozen after validation.")
        object.__setattr__(self, key, value)

    def __delattr__(self, key):
        if getattr(self, "_validated", False):
            raise RuntimeError("Cannot delete attributes of a validated config.")
        object.__delattr__(self, key)

    @contextlib.contextmanager
    def _set_implicit_default(self, _allow=True):
        yield

    # ------------------------------------------------------------------ validation
    def validate(self, *, _is_validating: bool = False):
        if not self._validated:
            try:
                self._validate()
            except (ValidationError, AssertionError, ValueError, TypeError, KeyError) as e:
                if _is_validating:
                    raise
                raise ValidationError(f"Validation failed for {type(self).__name__}: {e}") from e
            object.__setattr__(self, "_validated", True)
        return self

    def _validate(self) -> None:
        """Override to set derived defaults *before* calling `super()._validate()`, or to add checks after it."""
        if self._abstract:
            raise ValidationError(f"{type(self).__name__} is abstract")
        hints = self._type_hints()
        errors = []
        for name, field in self.__fields__.items():
            value = getattr(self, name)
            try:
                if value is MISSING:
                    value = self._default_for_missing(name, hints.get(name, typing.Any))
                value = _coerce(value, hints.get(name, typing.Any), f"{type(self).__name__}.{name}")
                if field.valid is not None:
                    value = field.valid(value)
            except (ValidationError, AssertionError, ValueError, TypeError, KeyError) as e:
                errors.append(f"{name}: {e}")
                continue
            object.__setattr__(self, name, value)
        if errors:
            raise ValidationError("; ".join(errors))
        if self.type is None and self._dynamic_type_names:
            object.__setattr__(self, "type", next(iter(self._dynamic_type_names.values())))

    def _default_for_missing(self, name: str, hint):
        cls = _config_class_of(hint)
        if cls is not None:
            cls = cls._get_default_subclass()
            return cls()
        raise ValidationError(f"Field {name} is required")

    # ------------------------------------------------------------------ (de)serialisation
    @classmethod
    def from_dict(cls, default: "Config | dict | None" = None, *updates: "Config | dict", strict: bool = True,
                  update_type: UpdateType = UpdateType.override):
        if isinstance(default, Config):
            default = default.to_dict()
        data = copy.deepcopy(default) if default else {}
        for update in updates:
            if isinstance(update, Config):
                update = update.to_dict(serialized=False)
            for key, value in update.items():
                set_nested_dict_value(data, key, value, update_type)
        return cls._from_dict(data, strict=strict)

    @classmethod
    def from_flat_dict(cls, default: dict, strict: bool = True):
        return cls._from_dict(copy.deepcopy(default), strict=strict, flat=True)

    @classmethod
    def _from_dict(cls, default: dict, strict: bool = True, flat: bool = False):
        if not isinstance(default, dict):
            raise ValidationError(f"Expected a dict for {cls.__name__}, got {type(default).__name__}")
        type_name = default.get("type")
        actual = cls
        if type_name is not None and isinstance(type_name, str):
            try:
                actual = cls.get_subclass(type_name)
            except KeyError:
                if cls.__dict__.get("_registry") is not None or any(b.__dict__.get("_registry") for b in cls.__mro__):
                    raise
        elif cls._abstract or cls.__dict__.get("_registry") is not None:
            actual = cls._get_default_subclass()
        if actual is not cls:
            return actual._from_dict(default, strict=strict, flat=flat)
        default = dict(default)
        cls._apply_renames(default)
        hints = cls._type_hints()
        kwargs = {}
        for name, field in cls.__fields__.items():
            if not field.init:
                continue
            hint = hints.get(name, typing.Any)
            if flat:
                sub = _config_class_of(hint)
                if sub is not None and name not in default:
                    kwargs[name] = sub._from_dict(default, strict=False, flat=True)
                    continue
            if name in default:
                kwargs[name] = _from_dict_value(default.pop(name), hint, strict)
        if strict and not flat and default:
            raise ValidationError(f"Unknown field(s) {sorted(default)} in {cls.__name__}")
        out = cls(**kwargs)
        if NoAutoValidate._depth == 0 and False:
            out.validate()
        return out

    @classmethod
    def _apply_renames(cls, default: dict) -> None:
        for base in cls.__mro__:
            for old, new in base.__dict__.get("_renamed_fields", {}).items():
                if old in default:
                    value = default.pop(old)
                    if callable(new):
                        new(default, value)
                    else:
                        logger.warning(f"Field `{old}` of {cls.__name__} is deprecated, use `{'.'.join(_as_tuple(new))}`")
                        set_nested_dict_value(default, new, value)

    def to_dict(self, verbose: int | None = FieldVerboseLevel.explicit, all_fields: bool = False,
                serialized: bool = True) -> dict:
        if verbose is not None:
            all_fields = True
        out = {}
        for name, field in self.__fields__.items():
            value = getattr(self, name)
            explicit = name in self._explicit_fields
            if isinstance(value, Config):
                nested = value.to_dict(verbose, all_fields, serialized)
                if nested or explicit:
                    out[name] = nested
                continue
            include = explicit
            if not include and all_fields and field.init and field.hint != FieldHint.derived:
                level = FieldHintImportance[field.hint]
                include = verbose is None or level <= verbose
            if not include and _contains_config(value):
                include = True
            if include and value is not MISSING:
                out[name] = _serialize(value, verbose, all_fields, serialized)
        if "type" not in out and self._dynamic_type_names and (all_fields or out):
            pass
        return out

    def to_copy(self, *updates, strict: bool = True, update_type: UpdateType = UpdateType.override):
        out = type(self).from_dict(self, *updates, strict=strict, update_type=update_type)
        if self._validated:
            out.validate()
        return out

    def to_serialized(self, verbose: int | None = FieldVerboseLevel.core) -> dict:
        return self.to_dict(verbose, serialized=True)

    def to_logs(self, verbose: int | None = FieldVerboseLevel.core, log_fn=logger.info, title: str | None = None,
                width: int = 80, fill_char: str = "-"):
        text = yaml.safe_dump(self.to_dict(verbose), sort_keys=False)
        title = title or type(self).__name__
        header = f" {title} ".center(width, fill_char)
        return log_fn(f"\n{header}\n{text}{fill_char * width}")

    def __repr__(self):
        return f"{type(self).__name__}({self.to_dict(FieldVerboseLevel.explicit, serialized=True)})"

    def __eq__(self, other):
        return type(self) is type(other) and self.to_dict(FieldVerboseLevel.everything) == other.to_dict(FieldVerboseLevel.everything)

    __hash__ = object.__hash__

    def compare(self, other: "Config", log_fn: typing.Callable | type[BaseException] = ValueError):
        errors = compare_nested(self.to_dict(FieldVerboseLevel.everything), other.to_dict(FieldVerboseLevel.everything))
        if errors:
            message = f"Config comparison errors ({type(self).__name__}):\n  " + "\n  ".join(errors)
            if isinstance(log_fn, type) and issubclass(log_fn, BaseException):
                raise log_fn(message)
            return log_fn(message)
        return None

    def save_yaml(self, path, verbose: int | None = FieldVerboseLevel.explicit) -> None:
        pathlib.Path(path).write_text(yaml.safe_dump(self.to_dict(verbose), sort_keys=False))

    @classmethod
    def load_yaml(cls, path, *updates, strict: bool = True):
        return cls.from_dict(yaml.safe_load(pathlib.Path(path).read_text()) or {}, *updates, strict=strict)


# The `type` field is attached after the class body so that the builtin `type` stays usable inside it.
_type_field = Field(default=None, desc="Name of the registered subclass to instantiate.", hint=FieldHint.feature)
_type_field.name = "type"
Config.__annotations__ = {**getattr(Config, "__annotations__", {}), "type": str | None}
Config.__own_fields__ = {"type": _type_field}
Config.__fields__ = {"type": _type_field}
Config.__type_hints_cache__ = None


class Configurable:
    """Mixin for objects built from a config: `Thing(config)` stores a validated config as `self._config`."""

    config_class: typing.ClassVar[type[Config]] = Config

    def __init__(self, config: Config, *args, **kwargs):
        Assert.custom(isinstance, config, self.config_class)
        config.validate()
        self._config = config
        super().__init__(*args, **kwargs)

    @property
    def config(self):
        return self._config


# ---------------------------------------------------------------------- helpers
def _as_tuple(key) -> tuple:
    if isinstance(key, str):
        return tuple(key.split("."))
    return tuple(key)


def set_nested_dict_value(d: dict, keys, value, update_type: UpdateType = UpdateType.override) -> None:
    keys = _as_tuple(keys)
    for key in keys[:-1]:
        nxt = d.get(key)
        if isinstance(nxt, Config):
            nxt = nxt.to_dict()
        if not isinstance(nxt, dict):
            nxt = {}
        d[key] = nxt
        d = nxt
    last = keys[-1]
    if isinstance(value, Config):
        value = value.to_dict()
    if update_type == UpdateType.update and isinstance(value, dict) and isinstance(d.get(last), dict):
        for k, v in value.items():
            set_nested_dict_value(d[last], (k,), v, update_type)
    else:
        d[last] = copy.deepcopy(value)


def get_nested_dict_value(d: dict, keys):
    for key in _as_tuple(keys):
        d = d[key]
    return d


def pop_nested_dict_value(d: dict, keys):
    keys = _as_tuple(keys)
    for key in keys[:-1]:
        d = d[key]
    return d.pop(keys[-1])


def _config_class_of(hint) -> type[Config] | None:
    """The Config subclass a type hint denotes (directly or as `X | None`), else None."""
    if isinstance(hint, type) and issubclass(hint, Config):
        return hint
    origin = typing.get_origin(hint)
    if origin is not None and isinstance(origin, type) and issubclass(origin, Config):
        return origin
    return None


def _union_args(hint):
    origin = typing.get_origin(hint)
    if origin is typing.Union or origin is types.UnionType:
        return typing.get_args(hint)
    return None


def _contains_config(value) -> bool:
    if isinstance(value, Config):
        return True
    if isinstance(value, dict):
        return any(_contains_config(v) for v in value.values())
    if isinstance(value, (list, tuple)):
        return any(_contains_config(v) for v in value)
    return False


def _from_dict_value(value, hint, strict: bool):
    """Turn nested dicts into Config instances where the type hint asks for one; leave other values for validation."""
    if isinstance(value, Config) or value is None:
        return value
    cls = _config_class_of(hint)
    if cls is not None:
        return cls._from_dict(value, strict=strict) if isinstance(value, dict) else value
    args = _union_args(hint)
    if args is not None:
        for arg in args:
            sub = _config_class_of(arg)
            if sub is not None and isinstance(value, dict):
                return sub._from_dict(value, strict=strict)
        for arg in args:
            if typing.get_origin(arg) in (dict, list, tuple, set):
                return _from_dict_value(value, arg, strict)
        return value
    origin = typing.get_origin(hint)
    targs = typing.get_args(hint)
    if origin is dict and isinstance(value, dict) and len(targs) == 2:
        return {k: _from_dict_value(v, targs[1], strict) for k, v in value.items()}
    if origin in (list, set) and isinstance(value, (list, tuple, set)) and targs:
        return [_from_dict_value(v, targs[0], strict) for v in value]
    if origin is tuple and isinstance(value, (list, tuple)) and targs:
        if len(targs) == 2 and targs[1] is Ellipsis:
            return tuple(_from_dict_value(v, targs[0], strict) for v in value)
        return tuple(_from_dict_value(v, t, strict) for v, t in zip(value, targs))
    return value


def _coerce(value, hint, path: str):
    """Validate `value` against `hint`, converting compatible representations (int->float, str->enum/path...)."""
    if hint is typing.Any or hint is None and value is None:
        return value
    if isinstance(hint, typing.TypeVar):
        return value
    args = _union_args(hint)
    if args is not None:
        if value is None and type(None) in args:
            return None
        errors = []
        # exact-type matches first so that e.g. `float | bool` keeps a bool a bool
        for arg in args:
            if arg is not type(None) and isinstance(arg, type) and type(value) is arg:
                return _coerce(value, arg, path)
        for arg in args:
            if arg is type(None):
                continue
            try:
                return _coerce(value, arg, path)
            except (ValidationError, AssertionError, ValueError, TypeError, KeyError) as e:
                errors.append(str(e))
        raise ValidationError(f"{path}: {value!r} matches none of {hint} ({'; '.join(errors)})")
    origin = typing.get_origin(hint)
    targs = typing.get_args(hint)
    if origin is type:
        target = targs[0] if targs else object
        if isinstance(value, str):
            resolver = getattr(target, "__fast_llm_from_name__", None)
            if resolver is None:
                raise ValidationError(f"{path}: cannot resolve class name {value!r}")
            value = resolver(value)
        if not (isinstance(value, type) and (target is object or issubclass(value, target))):
            raise ValidationError(f"{path}: expected a subclass of {target}, got {value!r}")
        return value
    if origin is dict:
        if not isinstance(value, dict):
            raise ValidationError(f"{path}: expected a dict, got {type(value).__name__}")
        if len(targs) == 2:
            return {_coerce(k, targs[0], path): _coerce(v, targs[1], f"{path}[{k}]") for k, v in value.items()}
        return value
    if origin is list:
        if not isinstance(value, (list, tuple)):
            raise ValidationError(f"{path}: expected a list, got {type(value).__name__}")
        return [_coerce(v, targs[0], f"{path}[{i}]") for i, v in enumerate(value)] if targs else list(value)
    if origin is set:
        if not isinstance(value, (list, tuple, set, frozenset)):
            raise ValidationError(f"{path}: expected a set, got {type(value).__name__}")
        return {_coerce(v, targs[0], path) for v in value} if targs else set(value)
    if origin is tuple:
        if not isinstance(value, (list, tuple)):
            raise ValidationError(f"{path}: expected a tuple, got {type(value).__name__}")
        if len(targs) == 2 and targs[1] is Ellipsis:
            return tuple(_coerce(v, targs[0], f"{path}[{i}]") for i, v in enumerate(value))
        if targs:
            if len(value) != len(targs):
                raise ValidationError(f"{path}: expected {len(targs)} entries, got {len(value)}")
            return tuple(_coerce(v, t, f"{path}[{i}]") for i, (v, t) in enumerate(zip(value, targs)))
        return tuple(value)
    if origin is not None:
        hint = origin
    if not isinstance(hint, type):
        return value
    if issubclass(hint, Config):
        if isinstance(value, dict):
            value = hint._from_dict(value)
        if value is None or value is MISSING:
            value = hint._get_default_subclass()()
        if not isinstance(value, hint):
            raise ValidationError(f"{path}: expected {hint.__name__}, got {type(value).__name__}")
        value.validate(_is_validating=True)
        return value
    if issubclass(hint, enum.Enum):
        if isinstance(value, hint):
            return value
        try:
            return hint(value)
        except ValueError:
            if isinstance(value, str) and value in hint.__members__:
                return hint[value]
            raise ValidationError(f"{path}: {value!r} is not a valid {hint.__name__} ({[m.value for m in hint]})")
    if hint is bool:
        if isinstance(value, bool):
            return value
        raise ValidationError(f"{path}: expected a bool, got {value!r}")
    if hint is int:
        if isinstance(value, bool):
            raise ValidationError(f"{path}: expected an int, got a bool")
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value.is_integer():
            return int(value)
        if isinstance(value, str):
            try:
                return int(value)
            except ValueError:
                pass
        raise ValidationError(f"{path}: expected an int, got {value!r}")
    if hint is float:
        if isinstance(value, bool):
            raise ValidationError(f"{path}: expected a float, got a bool")
        if isinstance(value, (int, float)):
            return float(value)
        if isinstance(value, str):
            try:
                return float(value)
            except ValueError:
                pass
        raise ValidationError(f"{path}: expected a float, got {value!r}")
    if hint is str:
        if isinstance(value, str):
            return value
        raise ValidationError(f"{path}: expected a str, got {value!r}")
    if issubclass(hint, pathlib.PurePath):
        if isinstance(value, (str, pathlib.PurePath)):
            return hint(value)
        raise ValidationError(f"{path}: expected a path, got {value!r}")
    converter = getattr(hint, "__fast_llm_coerce__", None)
    if converter is not None:
        return converter(value)
    if isinstance(value, hint):
        return value
    raise ValidationError(f"{path}: expected {hint.__name__}, got {type(value).__name__} ({value!r})")


def _serialize(value, verbose, all_fields, serialized):
    if isinstance(value, Config):
        return value.to_dict(verbose, all_fields, serialized)
    if isinstance(value, dict):
        return {(_serialize(k, verbose, all_fields, serialized)): _serialize(v, verbose, all_fields, serialized) for k, v in value.items()}
    if isinstance(value, (list, tuple, set, frozenset)):
        items = [_serialize(v, verbose, all_fields, serialized) for v in value]
        if isinstance(value, (set, frozenset)):
            items = sorted(items)
        return items
    if not serialized:
        return value
    if isinstance(value, enum.Enum):
        return value.value
    if isinstance(value, pathlib.PurePath):
        return str(value)
    if isinstance(value, type):
        serializer = getattr(value, "__fast_llm_serialize__", None)
        return serializer() if serializer else value.__name__
    if isinstance(value, (bool, int, float, str)) or value is None:
        return value
    serializer = getattr(value, "__fast_llm_serialize__", None)
    if serializer is not None:
        return serializer()
    return str(value)
