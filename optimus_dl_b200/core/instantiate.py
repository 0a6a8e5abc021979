"""Small ``_target_``-able helpers for config files (optimus_dl/core/instantiate.py:19-175).

Argument names and orders are the reference's (``cond(condition, true_val, false_val)``, ``repeat(times, item)``,
``get_item(key, mapping, default)``); the spellings this package used first (``if_true`` / ``if_false``, ``value``,
``obj``) are still accepted as keywords. Config nodes are turned into plain containers on the way in, so the results
can be passed on as ordinary keyword arguments.
"""

from __future__ import annotations

import copy
from collections.abc import Mapping
from typing import Any, Callable

from . import conf

_UNSET: Any = object()


def _plain(x: Any) -> Any:
    return conf.to_container(x, resolve=True) if conf.is_config(x) else x


def _deep_merge(dst: dict, src: Mapping) -> dict:
    for k, v in src.items():
        if isinstance(v, Mapping) and isinstance(dst.get(k), dict):
            _deep_merge(dst[k], v)
        else:
            dst[k] = copy.deepcopy(v)
    return dst


def merge_dicts(*dicts: Any, **extra: Any) -> dict:
    """Deep merge, later arguments win: ``merge_dicts({"b": {"c": 2}}, {"b": {"d": 3}}) == {"b": {"c": 2, "d": 3}}``."""
    out: dict = {}
    for d in dicts:
        if d is None:
            continue
        d = _plain(d)
        if not isinstance(d, Mapping):
            raise ValueError(f"Expected a mapping, but got {type(d).__name__}")
        _deep_merge(out, d)
    if extra:
        _deep_merge(out, {k: _plain(v) for k, v in extra.items()})
    return out


def cond(condition: Any, true_val: Any = _UNSET, false_val: Any = _UNSET, *, if_true: Any = _UNSET, if_false: Any = _UNSET) -> Any:
    """``true_val`` when ``condition`` holds, else ``false_val``: a switch between two sub-configs."""
    yes = true_val if true_val is not _UNSET else if_true
    no = false_val if false_val is not _UNSET else if_false
    picked = yes if condition else no
    return None if picked is _UNSET else _plain(picked)


def repeat(times: Any = _UNSET, item: Any = _UNSET, *, value: Any = _UNSET) -> list:
    """``times`` independent deep copies of ``item``."""
    if item is _UNSET:
        item = value
    if item is _UNSET or times is _UNSET:
        raise TypeError("repeat() needs 'times' and 'item'")
    if not isinstance(times, int) and isinstance(item, int) and not isinstance(item, bool):
        times, item = item, times          # the order this package used first: repeat(value, times)
    item = _plain(item)
    return [copy.deepcopy(item) for _ in range(int(times))]


def concat_lists(*lists: Any) -> list:
    out: list = []
    for l in lists:
        if l is None:                      # an optional list that was left out
            continue
        l = _plain(l)
        if isinstance(l, tuple):
            l = list(l)
        if not isinstance(l, list):
            raise ValueError(f"Expected a list, but got {type(l).__name__}")
        out.extend(l)
    return out


def get_item(key: Any = _UNSET, mapping: Any = _UNSET, default: Any = None, *, obj: Any = _UNSET) -> Any:
    """``mapping[key]``; ``default`` when the key is absent and a default (other than None) was given, else KeyError.
    Works as a switch in configs: ``key: ${args.kind}`` picks one of several sub-configs."""
    if mapping is _UNSET:
        mapping = obj
    if key is _UNSET or mapping is _UNSET:
        raise TypeError("get_item() needs 'key' and 'mapping'")
    key, mapping = _plain(key), _plain(mapping)
    if isinstance(key, (Mapping, list)) and not isinstance(mapping, (Mapping, list)):
        key, mapping = mapping, key        # the order this package used first: get_item(obj, key)
    try:
        return mapping[key]
    except (KeyError, IndexError, TypeError):
        pass
    if default is not None:
        return default
    raise KeyError(f"Key {key!r} not found in mapping and no default provided.")


def compose(*functions: Callable[..., Any]) -> Callable[..., Any]:
    """Left-to-right function composition: ``compose(f, g)(x) == g(f(x))``. The first function receives all the
    arguments of the call, each later one the previous result; with no functions the pipeline is the identity."""

    def run(*args: Any, **kwargs: Any) -> Any:
        if not functions:
            if len(args) == 1 and not kwargs:
                return args[0]
            raise ValueError("compose() of no functions takes exactly one positional argument")
        x = functions[0](*args, **kwargs)
        for f in functions[1:]:
            x = f(x)
        return x

    return run
