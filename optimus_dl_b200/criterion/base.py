"""Criterion interface (optimus_dl/modules/criterion/base.py:14-69)."""

from __future__ import annotations

from typing import Any

import torch


class BaseCriterion:
    """``criterion(model, batch, requested_protocols) -> (loss, exposed_protocols)``."""

    def __call__(self, model: torch.nn.Module, batch: dict[str, Any],
                 requested_protocols: set[str] | None = None) -> tuple[torch.Tensor, dict[str, Any]]:
        raise NotImplementedError
