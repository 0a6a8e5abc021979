"""Resolvers and lazy ``_target_`` instantiation for the config tree.

Counterpart of optimus_dl/core/omegaconf_utils.py in the reference: registers the ``eval``,
``cpu_count``, ``hash``, ``config_hash`` and ``oc.env`` / ``oc.select`` resolvers at import and
provides :func:`non_resolving_instantiate`, which turns every ``_target_`` node into a lazily
built object that (a) is only constructed when read, (b) is rebuilt when any value it
interpolates changes, and (c) detects dependency cycles. Interpolations elsewhere in the tree
are left unresolved, so ``cfg.b = "${.a}"`` keeps following ``cfg.a``.
"""

from __future__ import annotations

import hashlib
import math
import os
from typing import Any

from . import conf
from .conf import DictNode, LazyTarget, ListNode


def _eval_resolver(expr: Any, **_: Any) -> Any:
    import numpy
    import torch

    scope: dict[str, Any] = {"torch": torch, "numpy": numpy, "np": numpy, "math": math, "os": os}
    try:
        import scipy

        scope["scipy"] = scipy
    except ImportError:
        pass
    return eval(str(expr), scope)  # noqa: S307 - config files are trusted input, as in the reference


def _env_resolver(name: str, default: Any = conf.MISSING) -> Any:
    v = os.environ.get(str(name))
    if v is None:
        if default == conf.MISSING:
            raise conf.InterpolationError(f"environment variable {name!r} is not set and has no default")
        return default
    return conf._parse_scalar(v) if not isinstance(v, str) else v


def _hash_resolver(*args: Any) -> str:
    return hashlib.sha256("|".join(map(str, args)).encode()).hexdigest()[:16]


def _config_hash_resolver(*_: Any, _root_: Any = None, **__: Any) -> str:
    raw = conf.to_container(_root_, resolve=False) if _root_ is not None else {}
    return hashlib.sha256(repr(raw).encode()).hexdigest()[:16]


def _select_resolver(path: str, default: Any = None, _root_: Any = None, **_: Any) -> Any:
    return conf.select(_root_, str(path), default=default)


conf.register_resolver("eval", _eval_resolver)
conf.register_resolver("cpu_count", lambda: os.cpu_count() or 1)
conf.register_resolver("hash", _hash_resolver)
conf.register_resolver("config_hash", _config_hash_resolver, pass_context=True)
conf.register_resolver("oc.env", _env_resolver)
conf.register_resolver("oc.select", _select_resolver, pass_context=True)


def _convert(node: Any) -> Any:
    """Replace ``_target_`` dict nodes by LazyTarget markers, depth first."""
    if isinstance(node, DictNode):
        for k in list(node._data):
            raw = node._data[k]
            if isinstance(raw, (DictNode, ListNode)):
                _convert(raw)
                if isinstance(raw, DictNode) and "_target_" in raw._data:
                    node._data[k] = LazyTarget(raw)
    elif isinstance(node, ListNode):
        for i, raw in enumerate(node._items):
            if isinstance(raw, (DictNode, ListNode)):
                _convert(raw)
                if isinstance(raw, DictNode) and "_target_" in raw._data:
                    node._items[i] = LazyTarget(raw)
    return node


def _force(node: Any) -> None:
    if isinstance(node, DictNode):
        for k in list(node._data):
            raw = node._data[k]
            if isinstance(raw, LazyTarget):
                node._data[k] = conf._wrap(raw.get(), node, k)
            else:
                _force(raw)
    elif isinstance(node, ListNode):
        for i, raw in enumerate(node._items):
            if isinstance(raw, LazyTarget):
                node._items[i] = conf._wrap(raw.get(), node, i)
            else:
                _force(raw)


def non_resolving_instantiate(config: Any, lazy: bool = True) -> Any:
    """Instantiate every ``_target_`` node of ``config`` without resolving other interpolations.

    ``lazy=True`` (default) builds objects on first access and rebuilds them when their inputs
    change; ``lazy=False`` builds everything now and stores the objects in the tree.
    A root that is itself a ``_target_`` node is instantiated and returned directly.
    """
    cfg = conf.create(config) if not conf.is_config(config) else conf.create(config)
    if isinstance(cfg, DictNode) and "_target_" in cfg._data:
        _convert(cfg)
        built = LazyTarget(cfg).get()
        return conf.to_container(built, resolve=True) if conf.is_config(built) else built   # a plain dict / list at the root
    _convert(cfg)
    if not lazy:
        _force(cfg)
    return cfg


# public names of the resolvers, as the reference exports them (optimus_dl/core/omegaconf_utils.py:95-118)
hash_resolver = _hash_resolver
conf_hash_resolver = _config_hash_resolver
