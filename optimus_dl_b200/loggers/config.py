"""Logger config base (optimus_dl/modules/loggers/config.py): ``id`` defaults to the registry name."""

from __future__ import annotations

from dataclasses import dataclass, field

from ..core.registry import RegistryConfig


@dataclass
class MetricsLoggerConfig(RegistryConfig):
    enabled: bool = True
    id: str | None = "${._name}"
    tags: list[str] = field(default_factory=list)
    notes: str | None = None
