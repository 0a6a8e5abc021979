"""``cosine_annealing``: ``eta_min + (base - eta_min) * (1 + cos(pi * t / T)) / 2`` with ``T`` = total
training iterations (the ``T_max`` config key is kept for compatibility and, as in the
reference, not used; optimus_dl/modules/lr_scheduler/cosine_annealing.py:14-85)."""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from . import register_lr_scheduler
from .base import BaseLRScheduler, BaseLRSchedulerConfig


@dataclass
class CosineAnnealingLRConfig(BaseLRSchedulerConfig):
    T_max: int = 1000
    eta_min: float = 0.0
    last_epoch: int = -1


@register_lr_scheduler("cosine_annealing", CosineAnnealingLRConfig)
class CosineAnnealingLR(BaseLRScheduler):
    def __init__(self, cfg, optimizer, iterations: int, **kwargs: Any):
        super().__init__(optimizer)
        self.T_max = int(iterations)
        self.eta_min = float(cfg.eta_min)
        self._step_count = int(cfg.last_epoch) + 1
        self.set()

    def get_lr(self) -> list[float]:
        w = (1.0 + math.cos(math.pi * self._step_count / self.T_max)) / 2.0
        return [self.eta_min + (b - self.eta_min) * w for b in self.base_lrs]

    def state_dict(self) -> dict[str, Any]:
        return {**super().state_dict(), "T_max": self.T_max, "eta_min": self.eta_min}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.T_max = state_dict.get("T_max", self.T_max)
        self.eta_min = state_dict.get("eta_min", self.eta_min)
        super().load_state_dict(state_dict)
