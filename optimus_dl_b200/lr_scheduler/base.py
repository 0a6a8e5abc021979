"""Scheduler base (optimus_dl/modules/lr_scheduler/base.py:20-87): owns a step counter, the
per-group base rates captured at construction, and writes ``lr`` into the optimizer's groups."""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any

from ..core.registry import RegistryConfig


@dataclass
class BaseLRSchedulerConfig(RegistryConfig):
    """Flexible on purpose: config files may carry keys a given schedule does not read."""


class BaseLRScheduler(ABC):
    def __init__(self, optimizer: Any, **kwargs: Any):
        self.optimizer = optimizer
        self._step_count = 0
        self.base_lrs = [g["lr"] for g in optimizer.param_groups]

    @abstractmethod
    def get_lr(self) -> list[float]: ...

    def set(self) -> None:
        values = self.get_lr()
        groups = self.optimizer.param_groups
        if len(values) != len(groups):
            raise ValueError(f"{len(values)} learning rates for {len(groups)} parameter groups")
        for g, lr in zip(groups, values):
            g["lr"] = lr

    def step(self) -> None:
        self._step_count += 1
        self.set()

    def get_last_lr(self) -> list[float]:
        return [g["lr"] for g in self.optimizer.param_groups]

    @property
    def last_epoch(self) -> int:
        return self._step_count

    def state_dict(self) -> dict[str, Any]:
        return {"step_count": self._step_count, "base_lrs": list(self.base_lrs)}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self._step_count = state_dict["step_count"]
        self.base_lrs = list(state_dict["base_lrs"])
        self.set()
