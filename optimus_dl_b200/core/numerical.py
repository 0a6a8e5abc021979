"""Small numeric helpers (optimus_dl/core/numerical.py:9-50)."""

from __future__ import annotations

from typing import Any

import torch


def get_item(x: Any) -> Any:
    """Python scalar from a tensor / numpy scalar / number."""
    if isinstance(x, torch.Tensor):
        return x.item()
    if hasattr(x, "item") and callable(x.item):
        try:
            return x.item()
        except (ValueError, TypeError):
            return x
    return x


def safe_round(x: Any, ndigits: int | None = None) -> Any:
    x = get_item(x)
    if ndigits is None:
        return x
    try:
        return round(x, ndigits)
    except TypeError:
        return x
