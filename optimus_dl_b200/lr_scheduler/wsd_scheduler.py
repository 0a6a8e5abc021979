"""``wsd``: warmup - stable - decay (optimus_dl/modules/lr_scheduler/wsd_scheduler.py:14-234).

Factor of the base rate as a function of the step ``t`` (``N`` iterations, ``D = int(fract_decay * N)``
decay steps, ``H = N - D``):

* ``t < warmup``: linear from ``1 / init_div_factor`` to 1;
* ``t < H``: 1;
* ``t < N``: a decay shape from ``cooldown_start_lr_factor`` to ``final_lr_factor`` over progress
  ``x = (t - H) / D``: ``linear``, ``linear_pw`` (piecewise through the given waypoints), ``exp``
  (``final ** x``), ``cosine``, ``miror_cosine`` (linear mirrored about the cosine), ``square``, ``sqrt``;
* afterwards ``final_lr_factor``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from . import register_lr_scheduler
from .base import BaseLRScheduler, BaseLRSchedulerConfig

DECAY_TYPES = ("linear", "linear_pw", "exp", "cosine", "miror_cosine", "square", "sqrt")


@dataclass
class WSDSchedulerConfig(BaseLRSchedulerConfig):
    final_lr_factor: float = 0.0
    warmup_steps: int | None = 300
    warmup_steps_fraction: float | None = None
    init_div_factor: int = 100
    fract_decay: float = 0.1
    decay_type: str = "linear"
    sqrt_power: float = 0.5
    linear_pw_subdivisions: list[float] | None = None
    cooldown_start_lr_factor: float = 1.0


@register_lr_scheduler("wsd", WSDSchedulerConfig)
class WSDScheduler(BaseLRScheduler):
    def __init__(self, cfg, optimizer, iterations: int, **kwargs: Any):
        super().__init__(optimizer)
        warm = cfg.warmup_steps
        if warm is None:
            assert cfg.warmup_steps_fraction is not None, "Either warmup_steps or warmup_steps_fraction must be specified"
            warm = int(cfg.warmup_steps_fraction * iterations)
        if cfg.decay_type not in DECAY_TYPES:
            raise ValueError(f"decay_type {cfg.decay_type} is not in {list(DECAY_TYPES)}")
        self.iterations = int(iterations)
        self.warmup_steps = int(warm)
        self.final_lr_factor = float(cfg.final_lr_factor)
        self.init_div_factor = cfg.init_div_factor
        self.fract_decay = float(cfg.fract_decay)
        self.decay_type = cfg.decay_type
        self.sqrt_power = float(cfg.sqrt_power)
        self.linear_pw_subdivisions = list(cfg.linear_pw_subdivisions or [])
        self.cooldown_start_lr_factor = float(cfg.cooldown_start_lr_factor)
        self.n_anneal_steps = int(self.fract_decay * self.iterations)
        self.n_hold = self.iterations - self.n_anneal_steps
        self.set()

    def get_lr(self) -> list[float]:
        f = self._get_lr_factor(self._step_count)
        return [b * f for b in self.base_lrs]

    def _get_lr_factor(self, step: int) -> float:
        if step < self.warmup_steps:
            x = step / self.warmup_steps
            return x + (1.0 - x) / self.init_div_factor
        if step < self.n_hold:
            return 1.0
        if step < self.iterations:
            return self._decay((step - self.n_hold) / self.n_anneal_steps)
        return self.final_lr_factor

    def _decay(self, x: float) -> float:
        lo, hi = self.final_lr_factor, self.cooldown_start_lr_factor
        span = hi - lo
        kind = self.decay_type
        if kind == "linear":
            return lo + span * (1.0 - x)
        if kind == "exp":
            return lo ** x
        if kind == "cosine":
            return lo + span * (1.0 + math.cos(math.pi * x)) * 0.5
        if kind == "miror_cosine":
            cos_v = lo + span * (1.0 + math.cos(math.pi * x)) * 0.5
            lin_v = lo + span * (1.0 - x)
            return 2.0 * lin_v - cos_v
        if kind == "square":
            return lo + span * (1.0 - x * x)
        if kind == "sqrt":
            return lo + span * (1.0 - x ** self.sqrt_power)
        # linear_pw: straight segments through [start, *waypoints, final]
        pts = [hi, *self.linear_pw_subdivisions, lo]
        seg = 1.0 / (len(pts) - 1)
        k = min(int(math.floor(x / seg)), len(pts) - 2)
        local = (x - seg * k) / seg
        return pts[k] + (pts[k + 1] - pts[k]) * local

    def state_dict(self) -> dict[str, Any]:
        keys = ("iterations", "warmup_steps", "final_lr_factor", "init_div_factor", "fract_decay", "decay_type",
                "sqrt_power", "linear_pw_subdivisions", "cooldown_start_lr_factor", "n_anneal_steps", "n_hold")
        return {**super().state_dict(), **{k: getattr(self, k) for k in keys}}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        for k, v in state_dict.items():
            if k not in ("step_count", "base_lrs") and hasattr(self, k):
                setattr(self, k, v)
        super().load_state_dict(state_dict)
