"""``linear_warmup``: ramp from ``start_lr`` to the target rate over ``warmup_steps`` (or a fraction
of the run), then hold (optimus_dl/modules/lr_scheduler/linear_warmup.py:12-90)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from . import register_lr_scheduler
from .base import BaseLRScheduler, BaseLRSchedulerConfig


@dataclass
class LinearWarmupLRConfig(BaseLRSchedulerConfig):
    warmup_steps: int | None = None
    warmup_percent: float | None = 0.05
    target_lr: float | None = None
    start_lr: float = 0.0


@register_lr_scheduler("linear_warmup", LinearWarmupLRConfig)
class LinearWarmupLR(BaseLRScheduler):
    def __init__(self, cfg, optimizer, iterations: int, **kwargs: Any):
        super().__init__(optimizer)
        steps = cfg.warmup_steps
        if steps is None:
            if cfg.warmup_percent is None:
                raise ValueError("Either warmup_steps or warmup_percent must be set")
            steps = int(iterations * cfg.warmup_percent)
        self.warmup_steps = int(steps)
        self.start_lr = float(cfg.start_lr)
        self.target_lrs = [cfg.target_lr or b for b in self.base_lrs]
        self.set()

    def get_lr(self) -> list[float]:
        if self.warmup_steps == 0 or self._step_count > self.warmup_steps:
            return list(self.target_lrs)
        f = self._step_count / self.warmup_steps
        return [self.start_lr + (t - self.start_lr) * f for t in self.target_lrs]

    def state_dict(self) -> dict[str, Any]:
        return {**super().state_dict(), "warmup_steps": self.warmup_steps, "start_lr": self.start_lr,
                "target_lrs": list(self.target_lrs)}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.warmup_steps = state_dict["warmup_steps"]
        self.start_lr = state_dict["start_lr"]
        self.target_lrs = list(state_dict["target_lrs"])
        super().load_state_dict(state_dict)
