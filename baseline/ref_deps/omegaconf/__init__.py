"""Stand-in for the `omegaconf` package, for the reference arm of bench.py only.

The semantics (containers with lazy interpolation, merge, structured configs from dataclasses) come from
this repository's dependency-free config tree, loaded here by file path under a private module name so that
the `optimus_dl_b200` package itself is never imported in the reference arm's process.
"""

from __future__ import annotations

import dataclasses
import importlib.util
import os
import sys
from typing import Any

_here = os.path.dirname(os.path.abspath(__file__))
_conf_path = os.path.normpath(os.path.join(_here, "..", "..", "..", "optimus_dl_b200", "core", "conf.py"))
_spec = importlib.util.spec_from_file_location("_ref_deps_conf", _conf_path)
_conf = importlib.util.module_from_spec(_spec)
sys.modules["_ref_deps_conf"] = _conf
_spec.loader.exec_module(_conf)

MISSING = _conf.MISSING
II = _conf.II
DictConfig = _conf.DictNode
ListConfig = _conf.ListNode
Container = _conf.Node


def SI(s: str) -> str:
    return s


def _defaults_of(cls: Any) -> dict:
    fields = {}
    for f in dataclasses.fields(cls):
        if f.default is not dataclasses.MISSING:
            fields[f.name] = f.default
        elif f.default_factory is not dataclasses.MISSING:
            fields[f.name] = f.default_factory()
        else:
            fields[f.name] = MISSING
    return fields


def _structured(obj: Any) -> Any:
    """Config node from a dataclass type or instance; the node remembers the type so that a later merge can fill
    nested dataclass fields (declared ``X | None = None``) with X's defaults, as a structured config does."""
    cls = obj if isinstance(obj, type) else type(obj)
    if dataclasses.is_dataclass(cls):
        node = _conf.create(_defaults_of(cls) if isinstance(obj, type) else obj)
        node._flags["struct_type"] = cls
        return node
    return _conf.create(obj)


def _dataclass_in(hint: Any) -> Any:
    """The dataclass type inside ``X``, ``Optional[X]`` or ``X | None`` (None when there is none)."""
    import types
    import typing

    if isinstance(hint, type) and dataclasses.is_dataclass(hint):
        return hint
    if typing.get_origin(hint) in (typing.Union, types.UnionType):
        for a in typing.get_args(hint):
            if isinstance(a, type) and dataclasses.is_dataclass(a):
                return a
    return None


def _typed_fill(cls: Any, data: Any) -> Any:
    """``data`` (a plain mapping about to be merged into a node of dataclass type ``cls``) with every nested
    mapping that targets a dataclass-typed field completed from that dataclass's defaults."""
    import typing

    if not isinstance(data, dict) or cls is None:
        return data
    try:
        hints = typing.get_type_hints(cls)
    except Exception:  # noqa: BLE001
        return data
    out = dict(data)
    for k, v in data.items():
        sub = _dataclass_in(hints.get(k))
        if sub is not None and isinstance(v, dict):
            base = _conf.to_container(_conf.create(_defaults_of(sub)), resolve=False)
            base.update(_typed_fill(sub, v))
            out[k] = base
    return out


class OmegaConf:
    create = staticmethod(_conf.create)
    structured = staticmethod(_structured)
    is_config = staticmethod(_conf.is_config)
    is_dict = staticmethod(_conf.is_dict)
    is_list = staticmethod(_conf.is_list)
    to_yaml = staticmethod(_conf.to_yaml)
    select = staticmethod(_conf.select)
    update = staticmethod(_conf.update)
    resolve = staticmethod(_conf.resolve)
    load = staticmethod(_conf.load)
    has_resolver = staticmethod(_conf.has_resolver)

    @staticmethod
    def merge(*cfgs: Any) -> Any:
        nodes = [_structured(c) if dataclasses.is_dataclass(c) else c for c in cfgs]
        cls = nodes[0]._flags.get("struct_type") if _conf.is_config(nodes[0]) else None
        if cls is not None:
            nodes = [nodes[0]] + [
                _typed_fill(cls, _conf.to_container(n, resolve=False) if _conf.is_config(n) else n) for n in nodes[1:]]
        out = _conf.merge(*nodes)
        if cls is not None and _conf.is_config(out):
            out._flags["struct_type"] = cls
        return out

    @staticmethod
    def to_container(cfg: Any, resolve: bool = False, throw_on_missing: bool = False, **_: Any) -> Any:
        return _conf.to_container(cfg, resolve=resolve, throw_on_missing=throw_on_missing)

    @staticmethod
    def is_interpolation(node: Any, key: Any = None) -> bool:
        try:
            raw = node._get_raw(key) if key is not None else node
        except (KeyError, IndexError, AttributeError):
            return False
        return _conf.is_interpolation(raw)

    @staticmethod
    def register_new_resolver(name: str, resolver: Any, *, replace: bool = False, use_cache: bool = False) -> None:
        import inspect

        try:
            params = inspect.signature(resolver).parameters
        except (TypeError, ValueError):
            params = {}
        ctx = "_root_" in params or "_parent_" in params
        _conf.register_resolver(name, resolver, use_cache=use_cache, replace=True, pass_context=ctx)

    @staticmethod
    def get_cache(node: Any) -> dict:
        return node._cache

    @staticmethod
    def set_struct(node: Any, value: Any) -> None:
        node._flags["struct"] = value

    @staticmethod
    def set_readonly(node: Any, value: Any) -> None:
        node._flags["readonly"] = value


from . import errors  # noqa: E402
from . import _utils, basecontainer  # noqa: E402,F401
