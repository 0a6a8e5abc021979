"""Small ``_target_``-able helpers for config files (optimus_dl/core/instantiate.py:19-175)."""

from __future__ import annotations

import copy
from typing import Any, Callable

from . import conf


def _plain(x: Any) -> Any:
    return conf.to_container(x, resolve=True) if conf.is_config(x) else x


def merge_dicts(*dicts: Any, **extra: Any) -> dict:
    out: dict = {}
    for d in dicts:
        if d:
            out.update(_plain(d))
    out.update({k: _plain(v) for k, v in extra.items()})
    return out


def cond(condition: Any, if_true: Any = None, if_false: Any = None) -> Any:
    return _plain(if_true) if condition else _plain(if_false)


def repeat(value: Any, times: int) -> list:
    v = _plain(value)
    return [copy.deepcopy(v) for _ in range(int(times))]


def concat_lists(*lists: Any) -> list:
    out: list = []
    for l in lists:
        if l:
            out.extend(_plain(l))
    return out


def get_item(obj: Any, key: Any, default: Any = None) -> Any:
    o = _plain(obj)
    try:
        return o[key]
    except (KeyError, IndexError, TypeError):
        if hasattr(o, str(key)):
            return getattr(o, str(key))
        return default


def compose(*functions: Callable[[Any], Any]) -> Callable[[Any], Any]:
    """Left-to-right function composition: ``compose(f, g)(x) == g(f(x))``."""

    def run(x: Any) -> Any:
        for f in functions:
            x = f(x)
        return x

    return run
