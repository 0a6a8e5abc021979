"""Optimizer builder (optimus_dl/recipe/train/builders/optimizer_builder.py:47-74)."""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

from ....core.registry import RegistryConfig, make_registry
from ....metrics.common import log_averaged
from ....optim import build_optimizer

logger = logging.getLogger(__name__)


@dataclass
class OptimizerBuilderConfig(RegistryConfig):
    pass


class OptimizerBuilder:
    def __init__(self, cfg: Any = None, optimization_config: Any = None, **kwargs: Any):
        self.cfg, self.optimization_config = cfg, optimization_config

    def build_optimizer(self, params: Any, **kwargs: Any):
        opt = build_optimizer(self.optimization_config.optimizer, params=params, **kwargs)
        n = sum(p.numel() for g in opt.param_groups for p in g["params"] if p.requires_grad)
        # averaged over ranks, as optimus_dl/recipe/train/builders/optimizer_builder.py:63-72 logs it
        log_averaged("optimized_params", n)
        clip = self.optimization_config.get("clip_grad_norm")
        if clip and hasattr(opt, "set_max_norm"):
            opt.set_max_norm(float(clip))
        return opt


_R, register_optimizer_builder, build_optimizer_builder = make_registry("optimizer_builder")
register_optimizer_builder("base", OptimizerBuilderConfig)(OptimizerBuilder)
