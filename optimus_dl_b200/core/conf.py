"""A small, dependency-free configuration tree with OmegaConf-style semantics.

The reference builds on omegaconf + hydra (optimus_dl/core/registry.py:48,
optimus_dl/core/omegaconf_utils.py). Neither is a dependency here; this module gives the
subset that its config tree uses:

* ``DictNode`` / ``ListNode`` containers with attribute and item access, parent links and
  lazy interpolation: ``${a.b}`` (absolute), ``${.a}`` / ``${..a}`` (relative), nested
  ``${a.${b}}``, string templates ``"x-${a}"`` and resolvers ``${name:arg1,arg2}``.
* ``create``, ``merge``, ``select``, ``update``, ``to_container``, ``to_yaml``, ``MISSING`` and ``II``.
* ``register_resolver`` with an optional per-node cache.

Interpolations are resolved on access, never eagerly, so a node copied elsewhere keeps
tracking the value it points to.
"""

from __future__ import annotations

import copy
import re
from collections.abc import Iterator, Mapping, MutableMapping, MutableSequence, Sequence
from typing import Any, Callable

import yaml

MISSING = "???"


def II(path: str) -> str:
    """Interpolation shorthand: ``II("a.b") == "${a.b}"``."""
    return "${" + path + "}"


class ConfigError(Exception):
    pass


class MissingMandatoryValue(ConfigError):
    pass


class InterpolationError(ConfigError):
    pass


class CircularDependencyError(InterpolationError, ValueError):
    """Two lazily instantiated ``_target_`` blocks need each other."""


_RESOLVERS: dict[str, tuple[Callable[..., Any], bool, bool]] = {}


def register_resolver(name: str, fn: Callable[..., Any], *, use_cache: bool = False, replace: bool = True,
                      pass_context: bool = False) -> None:
    """Register ``${name:...}``. With ``pass_context`` the function also receives ``_parent_`` and ``_root_``."""
    if name in _RESOLVERS and not replace:
        raise ConfigError(f"resolver {name!r} already registered")
    _RESOLVERS[name] = (fn, use_cache, pass_context)


def has_resolver(name: str) -> bool:
    return name in _RESOLVERS


class Node:
    __slots__ = ("_parent", "_key", "_flags")

    def _root(self) -> "Node":
        n = self
        while n._parent is not None:
            n = n._parent
        return n

    def _full_key(self) -> str:
        parts = []
        n: Node | None = self
        while n is not None and n._parent is not None:
            parts.append(str(n._key))
            n = n._parent
        return ".".join(reversed(parts))


class LazyTarget:
    """A ``_target_`` definition that is instantiated on access and re-instantiated when the
    values it depends on change (its resolved arguments are fingerprinted)."""

    __slots__ = ("definition", "_value", "_fp", "_busy")

    def __init__(self, definition: "DictNode"):
        self.definition = definition
        self._value = None
        self._fp = None
        self._busy = False

    def get(self) -> Any:
        if self._busy:
            raise CircularDependencyError(f"Circular dependency detected while instantiating '{self.definition._full_key()}'")
        self._busy = True
        try:
            plain = to_container(self.definition, resolve=True)
            fp = _fingerprint(plain)
            if self._fp is None or fp != self._fp:
                self._value = _wrap_result(instantiate_plain(plain))
                self._fp = fp
            return self._value
        finally:
            self._busy = False

    def __deepcopy__(self, memo):
        return LazyTarget(copy.deepcopy(self.definition, memo))


def _fingerprint(obj: Any) -> Any:
    if isinstance(obj, dict):
        return tuple((k, _fingerprint(v)) for k, v in obj.items())
    if isinstance(obj, (list, tuple)):
        return tuple(_fingerprint(v) for v in obj)
    if isinstance(obj, (str, int, float, bool, type(None))):
        return obj
    return ("obj", id(obj))


def _wrap_result(v: Any) -> Any:
    if type(v) is dict:
        return DictNode(v)
    if type(v) is list:
        return ListNode(v)
    return v


def locate(path: str) -> Any:
    """Import ``pkg.mod.attr`` and return the attribute."""
    import importlib

    parts = path.split(".")
    for i in range(len(parts), 0, -1):
        try:
            obj = importlib.import_module(".".join(parts[:i]))
        except ImportError:
            continue
        for a in parts[i:]:
            obj = getattr(obj, a)
        return obj
    raise ImportError(f"cannot locate {path!r}")


def instantiate_plain(plain: Any) -> Any:
    """Instantiate a resolved ``{_target_, _args_, _partial_, **kwargs}`` dict (recursing into values)."""
    if isinstance(plain, list):
        return [instantiate_plain(v) for v in plain]
    if not isinstance(plain, dict):
        return plain
    if "_target_" not in plain:
        return {k: instantiate_plain(v) for k, v in plain.items()}
    target = plain["_target_"]
    fn = locate(target) if isinstance(target, str) else target
    args = [instantiate_plain(a) for a in plain.get("_args_", [])]
    kwargs = {k: instantiate_plain(v) for k, v in plain.items()
              if k not in ("_target_", "_args_", "_partial_", "_recursive_", "_convert_")}
    if plain.get("_partial_"):
        import functools

        return functools.partial(fn, *args, **kwargs)
    return fn(*args, **kwargs)


def _wrap(value: Any, parent: Node | None, key: Any) -> Any:
    if isinstance(value, LazyTarget):
        object.__setattr__(value.definition, "_parent", parent)
        object.__setattr__(value.definition, "_key", key)
        return value
    if isinstance(value, Node):
        if value._parent is not None and value._parent is not parent:
            value = copy.deepcopy(value)
        object.__setattr__(value, "_parent", parent)
        object.__setattr__(value, "_key", key)
        return value
    import dataclasses

    # dataclass instances first: flexible registry configs are dataclasses AND dict subclasses (their fields would be
    # lost if they were taken for plain mappings; _dataclass_to_dict adds the mapping's own items on top)
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        return DictNode(_dataclass_to_dict(value), parent=parent, key=key)
    if isinstance(value, Mapping):
        return DictNode(value, parent=parent, key=key)
    if isinstance(value, (list, tuple)):
        return ListNode(value, parent=parent, key=key)
    return value


def _dataclass_to_dict(obj: Any) -> dict:
    import dataclasses

    out = {}
    for f in dataclasses.fields(obj):
        v = getattr(obj, f.name)
        if dataclasses.is_dataclass(v) and not isinstance(v, type):
            v = _dataclass_to_dict(v)
        out[f.name] = v
    extra = getattr(obj, "_extra", None)
    if isinstance(obj, dict):
        out.update(obj)
    elif isinstance(extra, dict):
        out.update(extra)
    return out


class DictNode(Node, MutableMapping):
    __slots__ = ("_data", "_cache")

    def __init__(self, data: Mapping | None = None, parent: Node | None = None, key: Any = None):
        object.__setattr__(self, "_parent", parent)
        object.__setattr__(self, "_key", key)
        object.__setattr__(self, "_flags", {})
        object.__setattr__(self, "_data", {})
        object.__setattr__(self, "_cache", {})
        if data:
            for k, v in data.items():
                self._data[k] = _wrap(v, self, k)

    # raw access -----------------------------------------------------------
    def _get_raw(self, key: Any) -> Any:
        return self._data[key]

    def _set_raw(self, key: Any, value: Any) -> None:
        self._data[key] = _wrap(value, self, key)

    # mapping protocol -------------------------------------------------------
    def __getitem__(self, key: Any) -> Any:
        if key not in self._data:
            raise KeyError(key)
        return _resolve_value(self._data[key], self, key)

    def __setitem__(self, key: Any, value: Any) -> None:
        self._set_raw(key, value)

    def __delitem__(self, key: Any) -> None:
        del self._data[key]

    def __iter__(self) -> Iterator:
        return iter(self._data)

    def __len__(self) -> int:
        return len(self._data)

    def __contains__(self, key: Any) -> bool:
        return key in self._data

    def __getattr__(self, key: str) -> Any:
        if key.startswith("__"):
            raise AttributeError(key)
        try:
            return self[key]
        except KeyError:
            raise AttributeError(f"config has no key {key!r} (at '{self._full_key()}')") from None

    def __setattr__(self, key: str, value: Any) -> None:
        self._set_raw(key, value)

    def __delattr__(self, key: str) -> None:
        try:
            del self._data[key]
        except KeyError:
            raise AttributeError(key) from None

    def get(self, key: Any, default: Any = None) -> Any:
        if key in self._data:
            v = self[key]
            return default if v is None and default is not None else v
        return default

    def pop(self, key: Any, *default: Any) -> Any:
        if key in self._data:
            v = self[key]
            del self._data[key]
            return v
        if default:
            return default[0]
        raise KeyError(key)

    def keys(self):
        return self._data.keys()

    def items(self):
        return [(k, self[k]) for k in self._data]

    def values(self):
        return [self[k] for k in self._data]

    def __repr__(self) -> str:
        return f"DictNode({to_container(self, resolve=False)!r})"

    def __eq__(self, other: Any) -> bool:
        if isinstance(other, (DictNode, Mapping)):
            return to_container(self, resolve=True) == (to_container(other, resolve=True) if isinstance(other, Node) else dict(other))
        return NotImplemented

    def __deepcopy__(self, memo):
        new = DictNode(None)
        for k, v in self._data.items():
            new._data[k] = _wrap(copy.deepcopy(v, memo), new, k)
        return new

    def copy(self) -> "DictNode":
        """A detached copy of this subtree (what ``DictConfig.copy()`` gives); interpolations stay unresolved."""
        return copy.deepcopy(self)

    def __getstate__(self):
        return {"data": to_container(self, resolve=False)}

    def __setstate__(self, state):
        self.__init__(state["data"])


class ListNode(Node, MutableSequence):
    __slots__ = ("_items",)

    def __init__(self, data: Sequence | None = None, parent: Node | None = None, key: Any = None):
        object.__setattr__(self, "_parent", parent)
        object.__setattr__(self, "_key", key)
        object.__setattr__(self, "_flags", {})
        object.__setattr__(self, "_items", [])
        if data:
            for i, v in enumerate(data):
                self._items.append(_wrap(v, self, i))

    def _reindex(self) -> None:
        for i, v in enumerate(self._items):
            if isinstance(v, Node):
                object.__setattr__(v, "_key", i)

    def _get_raw(self, idx: int) -> Any:
        return self._items[idx]

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return [self[i] for i in range(*idx.indices(len(self._items)))]
        return _resolve_value(self._items[idx], self, idx if idx >= 0 else len(self._items) + idx)

    def __setitem__(self, idx, value):
        self._items[idx] = _wrap(value, self, idx)

    def __delitem__(self, idx):
        del self._items[idx]
        self._reindex()

    def __len__(self):
        return len(self._items)

    def insert(self, idx, value):
        self._items.insert(idx, _wrap(value, self, idx))
        self._reindex()

    def __iter__(self):
        for i in range(len(self._items)):
            yield self[i]

    def __repr__(self):
        return f"ListNode({to_container(self, resolve=False)!r})"

    def __eq__(self, other):
        if isinstance(other, (ListNode, list, tuple)):
            return to_container(self, resolve=True) == (to_container(other, resolve=True) if isinstance(other, Node) else list(other))
        return NotImplemented

    def __deepcopy__(self, memo):
        new = ListNode(None)
        for i, v in enumerate(self._items):
            new._items.append(_wrap(copy.deepcopy(v, memo), new, i))
        return new

    def copy(self) -> "ListNode":
        return copy.deepcopy(self)

    # concatenation with lists and other list nodes, as ``ListConfig`` allows (``[0.0] + cfg.points``); the result
    # is a detached list node of the resolved items
    def __add__(self, other: Any) -> "ListNode":
        if not isinstance(other, (list, tuple, ListNode)):
            return NotImplemented
        return ListNode(list(to_container(self, resolve=True)) + list(to_container(other, resolve=True)
                                                                     if isinstance(other, ListNode) else other))

    def __radd__(self, other: Any) -> "ListNode":
        if not isinstance(other, (list, tuple)):
            return NotImplemented
        return ListNode(list(other) + list(to_container(self, resolve=True)))

    def __getstate__(self):
        return {"data": to_container(self, resolve=False)}

    def __setstate__(self, state):
        self.__init__(state["data"])


# ----------------------------------------------------------------------------- interpolation
_SIMPLE = re.compile(r"^\$\{([^${}]+)\}$")


def _find_matching_quoted(s: str, start: int) -> int:
    """Index of the ``}`` that closes the ``${`` at ``start``, reading quoted text inside an interpolation as text:
    a ``}`` or ``{`` between quotes closes or opens nothing, while ``${...}`` between quotes is still an interpolation.
    Returns -1 when the quotes do not pair up (an apostrophe in an unquoted argument, say)."""
    ctx: list[str] = []                    # "$" for an open interpolation, else the quote character that is open
    i = start
    while i < len(s):
        if s.startswith("${", i):
            ctx.append("$")
            i += 2
            continue
        c = s[i]
        top = ctx[-1] if ctx else ""
        if top == "$":
            if c == "}":
                ctx.pop()
                if not ctx:
                    return i
            elif c in "\"'":
                ctx.append(c)
        elif top:
            if c == "\\" and i + 1 < len(s):
                i += 2
                continue
            if c == top:
                ctx.pop()
        i += 1
    return -1


def _find_matching(s: str, start: int) -> int:
    j = _find_matching_quoted(s, start)
    if j >= 0:
        return j
    depth = 0
    i = start
    while i < len(s):
        if s.startswith("${", i):
            depth += 1
            i += 2
            continue
        if s[i] == "}":
            depth -= 1
            if depth == 0:
                return i
        i += 1
    raise InterpolationError(f"unbalanced interpolation in {s!r}")


def is_interpolation(value: Any) -> bool:
    return isinstance(value, str) and "${" in value


def _split_args(s: str) -> list[str]:
    args, depth, cur = [], 0, []
    i = 0
    quote = None
    while i < len(s):
        c = s[i]
        if quote:
            cur.append(c)
            if c == quote:
                quote = None
        elif c in "\"'":
            quote = c
            cur.append(c)
        elif s.startswith("${", i):
            depth += 1
            cur.append("${")
            i += 2
            continue
        elif c in "([{":
            depth += 1
            cur.append(c)
        elif c in ")]}":
            depth -= 1
            cur.append(c)
        elif c == "," and depth == 0:
            args.append("".join(cur).strip())
            cur = []
        else:
            cur.append(c)
        i += 1
    if cur or args:
        args.append("".join(cur).strip())
    return args


def _parse_scalar(text: str) -> Any:
    t = text.strip()
    if len(t) >= 2 and t[0] == t[-1] and t[0] in "\"'":
        return t[1:-1]
    try:
        v = yaml.safe_load(t)
    except yaml.YAMLError:
        return t
    if isinstance(v, (dict, list)):
        return t
    return v if v is not None or t in ("null", "~", "") else t


def select_relative(container: Node, path: str, *, origin_key: Any = None, throw: bool = True, default: Any = None,
                    resolve: bool = True, _stack: tuple = ()) -> Any:
    """Resolve ``path`` (``a.b``, ``.a``, ``..a.b``, ``a[0]``) starting at ``container``."""
    node: Any = container
    p = path
    if p.startswith("."):
        dots = len(p) - len(p.lstrip("."))
        p = p[dots:]
        for _ in range(dots - 1):
            if node._parent is None:
                raise InterpolationError(f"relative path {path!r} climbs above the root")
            node = node._parent
    else:
        node = container._root()
    if p == "":
        return node
    tokens = [t for t in re.split(r"\.|\[|\]", p) if t != ""]
    for i, tok in enumerate(tokens):
        if isinstance(node, DictNode):
            key: Any = tok
            if key not in node._data:
                alt = _parse_scalar(tok)
                if alt in node._data:
                    key = alt
                else:
                    if throw:
                        raise InterpolationError(f"key {tok!r} not found while resolving {path!r} (at '{container._full_key()}')")
                    return default
            raw = node._data[key]
            if isinstance(raw, LazyTarget) and raw._busy and i < len(tokens) - 1:
                # a ``_target_`` block naming one of its own parameters by absolute path: read the definition
                node = raw.definition
            else:
                node = _resolve_value(raw, node, key, _stack) if (resolve or i < len(tokens) - 1) else raw
        elif isinstance(node, ListNode):
            try:
                idx = int(tok)
                raw = node._items[idx]
            except (ValueError, IndexError):
                if throw:
                    raise InterpolationError(f"bad list index {tok!r} while resolving {path!r}") from None
                return default
            node = _resolve_value(raw, node, idx, _stack) if (resolve or i < len(tokens) - 1) else raw
        else:
            if throw:
                raise InterpolationError(f"cannot descend into {type(node).__name__} at {tok!r} while resolving {path!r}")
            return default
    return node


def _resolve_expr(expr: str, container: Node, key: Any, stack: tuple) -> Any:
    """Resolve the inside of one ``${...}``."""
    # inner interpolations first (``${a.${b}}`` or resolver args)
    expr = expr.strip()
    colon = _top_level_colon(expr)
    if colon >= 0:
        name = expr[:colon].strip()
        raw_args = _split_args(expr[colon + 1:])
        if name not in _RESOLVERS:
            raise InterpolationError(f"unknown resolver {name!r}")
        fn, use_cache, pass_ctx = _RESOLVERS[name]
        args = []
        for a in raw_args:
            quoted = len(a) >= 2 and a[0] == a[-1] and a[0] in "\"'"
            inner = a[1:-1] if quoted else a
            if "${" in inner:
                v = _resolve_string(inner, container, key, stack)
                args.append(str(v) if quoted and not isinstance(v, str) else v)
            else:
                args.append(inner if quoted else _parse_scalar(a))
        kwargs = {}
        if pass_ctx:
            kwargs = {"_parent_": container, "_root_": container._root(), "_key_": key}
        if use_cache and isinstance(container, DictNode):
            ck = (name, tuple(map(repr, args)))
            cache = container._cache
            if ck not in cache:
                cache[ck] = fn(*args, **kwargs)
            return cache[ck]
        return fn(*args, **kwargs)
    if "${" in expr:
        expr = str(_resolve_string(expr, container, key, stack))
    return select_relative(container, expr, origin_key=key, _stack=stack)


def _top_level_colon(expr: str) -> int:
    depth = 0
    i = 0
    while i < len(expr):
        if expr.startswith("${", i):
            depth += 1
            i += 2
            continue
        c = expr[i]
        if c == "}":
            depth -= 1
        elif c == ":" and depth == 0:
            return i
        elif c in " \t" and depth == 0:
            pass
        i += 1
    return -1


def _resolve_string(s: str, container: Node, key: Any, stack: tuple) -> Any:
    ident = (id(container), key, s)
    if ident in stack:
        raise InterpolationError(f"circular interpolation while resolving {s!r} at '{container._full_key()}.{key}'")
    stack = stack + (ident,)
    # whole-string interpolation keeps the referenced type
    if s.startswith("${") and _find_matching(s, 0) == len(s) - 1:
        return _resolve_expr(s[2:-1], container, key, stack)
    out = []
    i = 0
    while i < len(s):
        if s.startswith("\\${", i):
            out.append("${")
            i += 3
            continue
        if s.startswith("${", i):
            j = _find_matching(s, i)
            v = _resolve_expr(s[i + 2:j], container, key, stack)
            if isinstance(v, Node):
                v = to_container(v, resolve=True)
            out.append(str(v))
            i = j + 1
        else:
            out.append(s[i])
            i += 1
    return "".join(out)


def _resolve_value(value: Any, container: Node, key: Any, stack: tuple = ()) -> Any:
    if isinstance(value, LazyTarget):
        return value.get()
    if isinstance(value, str):
        if value == MISSING:
            raise MissingMandatoryValue(f"missing mandatory value: '{container._full_key()}.{key}'".replace("'.", "'"))
        if "${" in value:
            return _resolve_string(value, container, key, stack)
    return value


# ----------------------------------------------------------------------------- public helpers
def create(obj: Any = None) -> Any:
    """Build a config tree from a dict / list / YAML string / dataclass instance."""
    if obj is None:
        return DictNode({})
    if isinstance(obj, str):
        obj = yaml.safe_load(obj)
        if obj is None:
            return DictNode({})
    if isinstance(obj, Node):
        return copy.deepcopy(obj)
    return _wrap(copy.deepcopy(obj) if isinstance(obj, (dict, list)) else obj, None, None)


def is_config(obj: Any) -> bool:
    return isinstance(obj, Node)


def is_dict(obj: Any) -> bool:
    return isinstance(obj, DictNode)


def is_list(obj: Any) -> bool:
    return isinstance(obj, ListNode)


def to_container(cfg: Any, resolve: bool = False, throw_on_missing: bool = False) -> Any:
    if isinstance(cfg, DictNode):
        out = {}
        for k, raw in cfg._data.items():
            out[k] = _item_to_container(cfg, k, raw, resolve, throw_on_missing)
        return out
    if isinstance(cfg, ListNode):
        return [_item_to_container(cfg, i, raw, resolve, throw_on_missing) for i, raw in enumerate(cfg._items)]
    if isinstance(cfg, Mapping):
        return {k: to_container(v, resolve, throw_on_missing) for k, v in cfg.items()}
    if isinstance(cfg, (list, tuple)):
        return [to_container(v, resolve, throw_on_missing) for v in cfg]
    return cfg


def _item_to_container(parent: Node, key: Any, raw: Any, resolve: bool, throw_on_missing: bool) -> Any:
    if isinstance(raw, LazyTarget):
        if resolve:
            v = raw.get()
            return to_container(v, resolve, throw_on_missing) if isinstance(v, Node) else v
        return to_container(raw.definition, False, throw_on_missing)
    if isinstance(raw, Node):
        return to_container(raw, resolve, throw_on_missing)
    if isinstance(raw, str):
        if raw == MISSING:
            if throw_on_missing:
                raise MissingMandatoryValue(f"missing mandatory value: {parent._full_key()}.{key}")
            return raw
        if resolve and "${" in raw:
            v = _resolve_string(raw, parent, key, ())
            return to_container(v, resolve, throw_on_missing) if isinstance(v, Node) else v
    return raw


def to_yaml(cfg: Any, resolve: bool = False) -> str:
    return yaml.safe_dump(to_container(cfg, resolve=resolve), sort_keys=False, default_flow_style=False)


def _merge_into(dst: DictNode, src: Any) -> None:
    src_items = src._data.items() if isinstance(src, DictNode) else src.items()
    for k, v in src_items:
        cur = dst._data.get(k)
        if isinstance(cur, DictNode) and isinstance(v, (DictNode, Mapping)):
            _merge_into(cur, v)
        else:
            dst._set_raw(k, copy.deepcopy(v))


def merge(*cfgs: Any) -> Any:
    """Right-most wins; dicts merge recursively, lists and scalars are replaced. Interpolations are kept."""
    cfgs = tuple(c for c in cfgs if c is not None)
    if not cfgs:
        return DictNode({})
    first = create(cfgs[0])
    if isinstance(first, ListNode):
        return create(cfgs[-1])
    for c in cfgs[1:]:
        c = c if isinstance(c, (Node, Mapping)) else create(c)
        _merge_into(first, c)
    return first


def select(cfg: Node, path: str, default: Any = None, throw_on_missing: bool = False) -> Any:
    try:
        return select_relative(cfg, path, throw=False, default=default)
    except MissingMandatoryValue:
        if throw_on_missing:
            raise
        return default


def update(cfg: Node, path: str, value: Any, force_add: bool = True) -> None:
    tokens = [t for t in re.split(r"\.|\[|\]", path) if t != ""]
    node: Any = cfg
    for tok in tokens[:-1]:
        if isinstance(node, DictNode):
            if tok not in node._data or not isinstance(node._data[tok], Node):
                if not force_add and tok not in node._data:
                    raise ConfigError(f"key {tok!r} not in config while updating {path!r}")
                node._set_raw(tok, {})
            node = node._data[tok]
        elif isinstance(node, ListNode):
            node = node._items[int(tok)]
        else:
            raise ConfigError(f"cannot descend into scalar at {tok!r} while updating {path!r}")
    last = tokens[-1]
    if isinstance(node, DictNode):
        if not force_add and last not in node._data:
            raise ConfigError(f"key {last!r} not in config while updating {path!r}")
        node._set_raw(last, value)
    elif isinstance(node, ListNode):
        node[int(last)] = value
    else:
        raise ConfigError(f"cannot set {path!r}")


def delete(cfg: Node, path: str) -> None:
    tokens = [t for t in re.split(r"\.|\[|\]", path) if t != ""]
    node: Any = cfg
    for tok in tokens[:-1]:
        node = node._data[tok] if isinstance(node, DictNode) else node._items[int(tok)]
    if isinstance(node, DictNode):
        if tokens[-1] not in node._data:
            raise ConfigError(f"cannot delete missing key {path!r}")
        del node._data[tokens[-1]]
    else:
        del node[int(tokens[-1])]


def resolve(cfg: Node) -> Node:
    """Return a copy with every interpolation replaced by its value."""
    return create(to_container(cfg, resolve=True))


def load(path: str) -> Any:
    with open(path) as f:
        return create(yaml.safe_load(f) or {})
