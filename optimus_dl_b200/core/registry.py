"""``_name``-keyed component registries with typed, dataclass-described configs.

Same public contract as optimus_dl/core/registry.py:52-606 in the reference:
``make_registry(name, base)`` returns ``(registry, register, build)``; ``@register("key", Cfg)``
stores ``(class, Cfg)`` and attaches ``cls.register_arch``; ``build(cfg, cast_to=None, **kw)``
accepts a string, dict, config node or dataclass instance, merges it over the dataclass
defaults, validates and casts it, and calls ``registered(cfg, **kw)``.
``RegistryConfigStrict`` rejects unknown keys, ``RegistryConfig`` keeps them.

The config handed to a component is a :class:`~optimus_dl_b200.core.conf.DictNode`
(attribute access, like an omegaconf ``DictConfig`` in the reference).
"""

from __future__ import annotations

import dataclasses
import enum
import functools
import logging
import types
import typing
from dataclasses import dataclass
from typing import Any, Callable, TypeVar, Union, get_args, get_origin, get_type_hints

from . import conf
from .conf import DictNode, ListNode

logger = logging.getLogger(__name__)

registries: dict[str, dict[str, tuple[Any, Any]]] = {}

T = TypeVar("T")


@dataclass
class RegistryConfigStrict:
    """Config base that only allows declared fields (plus ``_name``)."""

    _name: str | None = None

    def get(self, key: str, default: Any = None) -> Any:
        """Mapping-style read of a declared field, so that a component built directly from a config INSTANCE (not
        through its registry, which hands over a config node) can use the same ``cfg.get(...)`` calls."""
        return getattr(self, key) if key in getattr(self, "__dataclass_fields__", {}) else default


@dataclass
class RegistryConfig(dict):
    """Config base that also accepts arbitrary extra keys (kept as mapping items)."""

    _name: str | None = None

    def __post_init__(self) -> None:
        pass

    def get(self, key: str, default: Any = None) -> Any:
        """Extra keys first (mapping items), then declared fields, then ``default``."""
        if dict.__contains__(self, key):
            return dict.__getitem__(self, key)
        return getattr(self, key) if key in getattr(self, "__dataclass_fields__", {}) else default


class ConfigValidationError(ValueError, TypeError, AssertionError):
    """A config does not fit its dataclass: unknown key (the reference raises ValueError there, AssertionError
    when the key is met inside ``build``) or a value that cannot be cast (TypeError there); each of these
    ``except`` forms catches this class."""


def _is_registry_cfg(cls: Any) -> bool:
    return isinstance(cls, type) and (issubclass(cls, RegistryConfig) or issubclass(cls, RegistryConfigStrict))


def _type_name(tp: Any) -> str:
    return getattr(tp, "__name__", None) or str(tp)


def dataclass_defaults(cls: type) -> dict:
    """Field defaults of a dataclass type as a plain dict (missing defaults become ``???``)."""
    out: dict[str, Any] = {}
    for f in dataclasses.fields(cls):
        if f.default is not dataclasses.MISSING:
            v = f.default
        elif f.default_factory is not dataclasses.MISSING:  # type: ignore[misc]
            v = f.default_factory()  # type: ignore[misc]
        else:
            v = conf.MISSING
        if dataclasses.is_dataclass(v) and not isinstance(v, type):
            v = instance_to_dict(v)
        out[f.name] = v
    return out


def instance_to_dict(obj: Any) -> dict:
    out: dict[str, Any] = {}
    for f in dataclasses.fields(obj):
        v = getattr(obj, f.name)
        if dataclasses.is_dataclass(v) and not isinstance(v, type):
            v = instance_to_dict(v)
        elif isinstance(v, (list, tuple)):
            v = [instance_to_dict(x) if dataclasses.is_dataclass(x) and not isinstance(x, type) else x for x in v]
        elif isinstance(v, enum.Enum):
            v = v
        out[f.name] = v
    if isinstance(obj, dict):
        for k, v in obj.items():
            out[k] = v
    return out


def _hints(cls: type) -> dict[str, Any]:
    try:
        return get_type_hints(cls)
    except Exception:  # unresolved forward references: fall back to raw annotations
        return {f.name: f.type for f in dataclasses.fields(cls)}


def _validate_and_cast(tp: Any, value: Any, path: str = "") -> Any:
    """Recursively check ``value`` against the type ``tp`` and cast where it is safe.

    Handles dataclasses, ``Optional``/``Union``, ``list``/``tuple``/``dict`` generics, enums and
    primitives (``"1e-3"`` -> float, ``3`` -> ``3.0``, ``"true"`` -> bool). Interpolation strings
    and the ``???`` marker pass through untouched.
    """
    if tp is Any or tp is None or tp is dataclasses.MISSING:
        return value
    if isinstance(value, str) and (conf.is_interpolation(value) or value == conf.MISSING):
        return value
    origin = get_origin(tp)
    if origin is Union or origin is types.UnionType:
        args = get_args(tp)
        if value is None and type(None) in args:
            return None
        errors = []
        # the first member the value can be cast to wins ("123" for int | str is 123), as in
        # optimus_dl/core/registry.py's union handling
        for a in args:
            if a is type(None):
                continue
            try:
                return _validate_and_cast(a, value, path)
            except ConfigValidationError as e:
                errors.append(str(e))
        raise ConfigValidationError(f"{path or 'value'}: {value!r} matches none of {_type_name(tp)} ({'; '.join(errors)})")
    if value is None:
        raise ConfigValidationError(f"{path or 'value'}: None is not allowed for {_type_name(tp)}")
    if dataclasses.is_dataclass(tp) and isinstance(tp, type):
        if dataclasses.is_dataclass(value) and not isinstance(value, type):
            value = instance_to_dict(value)
        if isinstance(value, (DictNode, dict)):
            raw = conf.to_container(value, resolve=False) if isinstance(value, DictNode) else dict(value)
            merged = dict(dataclass_defaults(tp))
            hints = _hints(tp)
            flexible = issubclass(tp, dict)
            for k, v in raw.items():
                if k not in hints and k != "_name" and not flexible:
                    raise ConfigValidationError(f"Unknown keys for {tp.__name__}: {path + '.' if path else ''}{k}")
                merged[k] = _deep_merge(merged.get(k), v)
            for k in list(merged):
                if k in hints:
                    merged[k] = _validate_and_cast(hints[k], merged[k], f"{path + '.' if path else ''}{k}")
            return merged
        raise ConfigValidationError(f"{path or 'value'}: expected mapping for {tp.__name__}, got {type(value).__name__}")
    if origin in (list, typing.List) or tp is list:
        if isinstance(value, (list, tuple, ListNode)):
            (et,) = get_args(tp) or (Any,)
            return [_validate_and_cast(et, v, f"{path}[{i}]") for i, v in enumerate(_raw_list(value))]
        raise ConfigValidationError(f"{path or 'value'}: expected list, got {type(value).__name__}")
    if origin in (tuple, typing.Tuple) or tp is tuple:
        if isinstance(value, (list, tuple, ListNode)):
            args = get_args(tp)
            vals = _raw_list(value)
            if args and args[-1] is not Ellipsis:
                if len(args) != len(vals):
                    raise ConfigValidationError(f"{path or 'value'}: expected {len(args)} items, got {len(vals)}")
                return [_validate_and_cast(a, v, f"{path}[{i}]") for i, (a, v) in enumerate(zip(args, vals))]
            et = args[0] if args else Any
            return [_validate_and_cast(et, v, f"{path}[{i}]") for i, v in enumerate(vals)]
        raise ConfigValidationError(f"{path or 'value'}: expected tuple, got {type(value).__name__}")
    if origin in (dict, typing.Dict) or tp is dict:
        if isinstance(value, (dict, DictNode)):
            args = get_args(tp)
            vt = args[1] if len(args) == 2 else Any
            raw = conf.to_container(value, resolve=False) if isinstance(value, DictNode) else value
            return {k: _validate_and_cast(vt, v, f"{path}.{k}") for k, v in raw.items()}
        if dataclasses.is_dataclass(value) and not isinstance(value, type):
            return instance_to_dict(value)
        raise ConfigValidationError(f"{path or 'value'}: expected dict, got {type(value).__name__}")
    if isinstance(tp, type) and issubclass(tp, enum.Enum):
        if isinstance(value, tp):
            return value
        for member in tp:
            if value == member.value or (isinstance(value, str) and value.lower() == member.name.lower()):
                return member
        raise ConfigValidationError(f"{path or 'value'}: {value!r} is not a member of {tp.__name__}")
    if tp is bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, str) and value.lower() in ("true", "false", "yes", "no", "on", "off", "1", "0"):
            return value.lower() in ("true", "yes", "on", "1")
        if isinstance(value, int) and value in (0, 1):
            return bool(value)
        raise ConfigValidationError(f"{path or 'value'}: {value!r} is not a bool")
    if tp is int:
        if isinstance(value, bool):
            raise ConfigValidationError(f"{path or 'value'}: bool is not an int")
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value.is_integer():
            return int(value)
        if isinstance(value, str):
            try:
                return int(value)
            except ValueError:
                pass
        raise ConfigValidationError(f"{path or 'value'}: {value!r} is not an int")
    if tp is float:
        if isinstance(value, bool):
            raise ConfigValidationError(f"{path or 'value'}: bool is not a float")
        if isinstance(value, (int, float)):
            return float(value)
        if isinstance(value, str):
            try:
                return float(value)
            except ValueError:
                pass
        raise ConfigValidationError(f"{path or 'value'}: {value!r} is not a float")
    if tp is str:
        if isinstance(value, str):
            return value
        if isinstance(value, (int, float, bool)):
            return str(value)
        raise ConfigValidationError(f"{path or 'value'}: {value!r} is not a str")
    if origin is typing.Literal:
        if value in get_args(tp):
            return value
        raise ConfigValidationError(f"{path or 'value'}: {value!r} not in {get_args(tp)}")
    return value



def validate_and_cast(tp: Any, value: Any, path: str = "") -> Any:
    """Check ``value`` against the type ``tp`` and cast where it is safe (see ``_validate_and_cast``).

    For a dataclass type the result is a config node: attribute and item access, extra keys of flexible configs kept
    (``casted.simple.param_int``, ``casted["extra"]``), as optimus_dl/core/registry.py:96-257 returns an OmegaConf
    object. Interpolations in a config node are resolved first.
    """
    if isinstance(value, conf.Node):
        value = conf.to_container(value, resolve=True)
    out = _validate_and_cast(tp, value, path)
    if dataclasses.is_dataclass(tp) and isinstance(tp, type) and isinstance(out, dict):
        return conf.create(out)
    return out

def _raw_list(v: Any) -> list:
    if isinstance(v, ListNode):
        return conf.to_container(v, resolve=False)
    return list(v)


def _deep_merge(base: Any, new: Any) -> Any:
    if isinstance(base, dict) and isinstance(new, dict):
        out = dict(base)
        for k, v in new.items():
            out[k] = _deep_merge(out.get(k), v)
        return out
    return new


def _get_cfg_path(cfg: Any) -> str:
    if isinstance(cfg, conf.Node):
        return cfg._full_key()
    return ""


def normalize_cfg(cfg: Any) -> dict | None:
    """Turn any accepted config form into a plain dict with interpolations resolved."""
    if cfg is None:
        return None
    if isinstance(cfg, str):
        return {"_name": cfg}
    if isinstance(cfg, conf.Node):
        return conf.to_container(cfg, resolve=True)
    if dataclasses.is_dataclass(cfg) and not isinstance(cfg, type):
        return instance_to_dict(cfg)
    if isinstance(cfg, dict):
        return conf.to_container(conf.create(cfg), resolve=True)
    raise TypeError(f"cannot build from config of type {type(cfg).__name__}")


def make_registry(registry_name: str, base_class: type | None = None):
    """Create (or fetch) the registry ``registry_name``; returns ``(dict, register, build)``."""
    registry = registries.setdefault(registry_name, {})

    def register_arch(name: str, class_name: str, registered_class: type):
        def wrapper(fn: Callable[[], Any]):
            arch = f"{class_name}-{name}"
            assert arch not in registry, f"Double registering of {arch} in {registry_name} registry"
            cfg_inst = fn()
            registry[arch] = (registered_class, cfg_inst)
            return fn

        return wrapper

    def register(name: str, cfg: type | None = None):
        assert name not in registry, f"Double registering of {name} in {registry_name} registry"
        assert cfg is None or _is_registry_cfg(cfg), "Configs must be subclasses of RegistryConfig or RegistryConfigStrict"

        def wrapper(registered_class):
            registry[name] = (registered_class, cfg)
            try:
                setattr(registered_class, "register_arch",
                        functools.partial(register_arch, class_name=name, registered_class=registered_class))
            except (AttributeError, TypeError):
                pass
            return registered_class

        return wrapper

    def build(cfg: Any, cast_to: type | None = None, **kwargs: Any) -> Any:
        if cfg is None:
            return None
        path = _get_cfg_path(cfg)
        raw = normalize_cfg(cfg)
        name = raw.get("_name") if raw else None
        if name is None:
            raise ValueError(f"config at '{path}' for registry '{registry_name}' has no _name: {raw!r}")
        if name not in registry:
            raise KeyError(f"'{name}' is not registered in registry '{registry_name}' (known: {sorted(registry)})")
        registered_class, cfg_spec = registry[name]
        if cfg_spec is None:
            merged = conf.create(raw)
        else:
            if isinstance(cfg_spec, type):
                cfg_cls, base = cfg_spec, {}
            else:  # register_arch stores a config *instance* with the arch's defaults
                cfg_cls, base = type(cfg_spec), instance_to_dict(cfg_spec)
            user = {k: v for k, v in raw.items() if not (k == "_name" and not isinstance(cfg_spec, type))}
            data = _deep_merge(base, user) if base else user
            try:
                merged = conf.create(validate_and_cast(cfg_cls, data, path))
            except ConfigValidationError as e:
                raise ConfigValidationError(f"invalid config for '{name}' in registry '{registry_name}': {e}") from None
            if merged.get("_name") is None:
                merged["_name"] = name
        obj = registered_class(merged, **kwargs)
        if cast_to is not None:
            assert isinstance(obj, cast_to), f"{type(obj).__name__} is not a {cast_to.__name__}"
        if base_class is not None and isinstance(registered_class, type):
            assert isinstance(obj, base_class), f"{type(obj).__name__} is not a {base_class.__name__}"
        return obj

    return registry, register, build


def build(registry_name: str, cfg: Any, cast_to: type | None = None, **kwargs: Any) -> Any:
    """Build from the named registry (module-level convenience, as in the reference)."""
    if registry_name not in registries:
        raise KeyError(f"unknown registry '{registry_name}' (known: {sorted(registries)})")
    _, _, builder = make_registry(registry_name)
    return builder(cfg, cast_to=cast_to, **kwargs)
