"""Transform config base (optimus_dl/modules/model_transforms/config.py:6-10)."""

from __future__ import annotations

from dataclasses import dataclass

from ..core.registry import RegistryConfig


@dataclass
class ModelTransformConfig(RegistryConfig):
    pass
