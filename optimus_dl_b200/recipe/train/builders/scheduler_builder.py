"""LR scheduler builder (optimus_dl/recipe/train/builders/scheduler_builder.py:49-70)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ....core.registry import RegistryConfig, make_registry
from ....lr_scheduler import build_lr_scheduler


@dataclass
class SchedulerBuilderConfig(RegistryConfig):
    pass


class SchedulerBuilder:
    def __init__(self, cfg: Any = None, lr_scheduler_config: Any = None, optimization_config: Any = None, **kwargs: Any):
        self.cfg, self.lr_scheduler_config, self.optimization_config = cfg, lr_scheduler_config, optimization_config

    def build_lr_scheduler(self, optimizer: Any, **kwargs: Any):
        if self.lr_scheduler_config is None:
            return None
        return build_lr_scheduler(self.lr_scheduler_config, optimizer=optimizer,
                                  iterations=int(self.optimization_config.iterations), **kwargs)


_R, register_scheduler_builder, build_scheduler_builder = make_registry("scheduler_builder")
register_scheduler_builder("base", SchedulerBuilderConfig)(SchedulerBuilder)
