"""Base model config (optimus_dl/modules/model/config.py)."""

from __future__ import annotations

from dataclasses import dataclass

from ..core.registry import RegistryConfigStrict


@dataclass
class ModelConfig(RegistryConfigStrict):
    pass
