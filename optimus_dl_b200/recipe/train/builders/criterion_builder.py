"""Criterion builder (optimus_dl/recipe/train/builders/criterion_builder.py:42-47)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ....core.registry import RegistryConfig, make_registry
from ....criterion import build_criterion


@dataclass
class CriterionBuilderConfig(RegistryConfig):
    pass


class CriterionBuilder:
    def __init__(self, cfg: Any = None, criterion_config: Any = None, **kwargs: Any):
        self.cfg, self.criterion_config = cfg, criterion_config

    def build_criterion(self, collective: Any = None, **kwargs: Any):
        return build_criterion(self.criterion_config, collective=collective, **kwargs)


_R, register_criterion_builder, build_criterion_builder = make_registry("criterion_builder")
register_criterion_builder("base", CriterionBuilderConfig)(CriterionBuilder)
