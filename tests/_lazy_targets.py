"""Importable targets for the lazy-instantiation tests (resolved by dotted path, so they live in a module of their own)."""

COUNT = {"n": 0}


def make(**kw):
    """Remembers how often it ran."""
    COUNT["n"] += 1
    return dict(kw, _call=COUNT["n"])


def add(a, b=0):
    return a + b
