"""Base config of criteria (optimus_dl/modules/criterion/config.py)."""

from __future__ import annotations

from dataclasses import dataclass

from ..core.registry import RegistryConfig


@dataclass
class CriterionConfig(RegistryConfig):
    pass
