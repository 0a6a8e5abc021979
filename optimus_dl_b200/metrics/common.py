"""Concrete meters and the ``log_*`` helpers (optimus_dl/modules/metrics/common.py:29-856)."""

from __future__ import annotations

import math
import time
from typing import Any, Callable

from ..core.numerical import safe_round
from .base import BaseMeter, log_meter


class AverageMeter(BaseMeter):
    def __init__(self, round: int | None = None):
        self.round, self.sum, self.count = round, 0.0, 0.0

    def log(self, value: float, weight: float = 1.0) -> None:
        self.sum += value * weight
        self.count += weight

    def compute(self) -> float:
        return safe_round(self.sum / self.count, self.round) if self.count else 0.0

    def merge(self, other_state: dict[str, Any]) -> None:
        self.sum += other_state["sum"]
        self.count += other_state["count"]


class SummedMeter(BaseMeter):
    def __init__(self, round: int | None = None):
        self.round, self.sum = round, 0.0

    def log(self, value: float) -> None:
        self.sum += value

    def compute(self) -> float:
        return safe_round(self.sum, self.round)

    def merge(self, other_state: dict[str, Any]) -> None:
        self.sum += other_state["sum"]


class MaxMeter(BaseMeter):
    def __init__(self, round: int | None = None):
        self.round, self.value = round, None

    def log(self, value: float) -> None:
        self.value = value if self.value is None else max(self.value, value)

    def compute(self) -> float:
        return safe_round(self.value, self.round) if self.value is not None else 0.0

    def merge(self, other_state: dict[str, Any]) -> None:
        if other_state["value"] is not None:
            self.log(other_state["value"])


class MinMeter(MaxMeter):
    def log(self, value: float) -> None:
        self.value = value if self.value is None else min(self.value, value)


class FrequencyMeter(BaseMeter):
    """Mean time between occurrences of an event, in milliseconds."""

    def __init__(self, round: int | None = None):
        self.round, self.total_ms, self.count, self._last = round, 0.0, 0, None

    def log(self) -> None:
        now = time.perf_counter()
        if self._last is not None:
            self.total_ms += (now - self._last) * 1e3
            self.count += 1
        self._last = now

    def compute(self) -> float:
        return safe_round(self.total_ms / self.count, self.round) if self.count else 0.0

    def merge(self, other_state: dict[str, Any]) -> None:
        self.total_ms += other_state["total_ms"]
        self.count += other_state["count"]

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        super().load_state_dict(state_dict)
        self._last = None  # wall-clock anchors do not survive a restart


class StopwatchMeter(BaseMeter):
    """Mean duration between ``start`` and ``end`` events, in milliseconds."""

    def __init__(self, round: int | None = None):
        self.round, self.total_ms, self.count, self._t0 = round, 0.0, 0, None

    def log(self, mode: str) -> None:
        if mode == "start":
            self.start()
        elif mode == "end":
            self.end()
        else:
            raise ValueError(f"unknown stopwatch mode {mode!r}")

    def start(self) -> None:
        self._t0 = time.perf_counter()

    def end(self) -> None:
        if self._t0 is not None:
            self.total_ms += (time.perf_counter() - self._t0) * 1e3
            self.count += 1
            self._t0 = None

    def compute(self) -> float:
        return safe_round(self.total_ms / self.count, self.round) if self.count else 0.0

    def merge(self, other_state: dict[str, Any]) -> None:
        self.total_ms += other_state["total_ms"]
        self.count += other_state["count"]

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        super().load_state_dict(state_dict)
        self._t0 = None


class AveragedExponentMeter(BaseMeter):
    """``exp(weighted mean(value))`` — perplexity from mean loss."""

    def __init__(self, round: int | None = None):
        self.round, self.sum, self.count = round, 0.0, 0.0

    def log(self, value: float, weight: float = 1.0) -> None:
        self.sum += value * weight
        self.count += weight

    def compute(self) -> float:
        if not self.count:
            return 0.0
        try:
            return safe_round(math.exp(self.sum / self.count), self.round)
        except OverflowError:
            return float("inf")

    def merge(self, other_state: dict[str, Any]) -> None:
        self.sum += other_state["sum"]
        self.count += other_state["count"]


class GatherMeter(BaseMeter):
    def __init__(self):
        self.values: list[Any] = []

    def log(self, value: Any) -> None:
        self.values.append(value)

    def compute(self) -> list[Any]:
        return list(self.values)

    def merge(self, other_state: dict[str, Any]) -> None:
        self.values.extend(other_state["values"])


def log_averaged(name: str, value: Any, weight: Any = 1.0, round: int | None = None, reset: bool = True,
                 priority: int = 100) -> None:
    log_meter(name, lambda: AverageMeter(round=round), reset=reset, priority=priority, value=value, weight=weight)


def log_averaged_exponent(name: str, value: Any, weight: Any = 1.0, round: int | None = None, reset: bool = True,
                          priority: int = 100) -> None:
    log_meter(name, lambda: AveragedExponentMeter(round=round), reset=reset, priority=priority, value=value, weight=weight)


def log_summed(name: str, value: Any, round: int | None = None, reset: bool = True, priority: int = 100) -> None:
    log_meter(name, lambda: SummedMeter(round=round), reset=reset, priority=priority, value=value)


def log_max(name: str, value: Any, round: int | None = None, reset: bool = True, priority: int = 100) -> None:
    log_meter(name, lambda: MaxMeter(round=round), reset=reset, priority=priority, value=value)


def log_min(name: str, value: Any, round: int | None = None, reset: bool = True, priority: int = 100) -> None:
    log_meter(name, lambda: MinMeter(round=round), reset=reset, priority=priority, value=value)


def log_event_start(name: str, round: int | None = None, reset: bool = True, priority: int = 100) -> None:
    log_meter(name, lambda: StopwatchMeter(round=round), reset=reset, priority=priority, force_log=True, mode="start")


def log_event_end(name: str, round: int | None = None, reset: bool = True, priority: int = 100) -> None:
    log_meter(name, lambda: StopwatchMeter(round=round), reset=reset, priority=priority, force_log=True, mode="end")


def log_event_occurence(name: str, round: int | None = None, reset: bool = True, priority: int = 100) -> None:
    log_meter(name, lambda: FrequencyMeter(round=round), reset=reset, priority=priority, force_log=True)


def log_gathered(name: str, value: Any, reset: bool = True, priority: int = 100) -> None:
    log_meter(name, GatherMeter, reset=reset, priority=priority, value=value)


class CachedLambda:
    """Callable evaluated at most once; lets several meters share one expensive value."""

    _UNSET = object()

    def __init__(self, func: Callable[[], Any]):
        self.func = func
        self._value: Any = self._UNSET

    def __call__(self) -> Any:
        if self._value is self._UNSET:
            self._value = self.func()
        return self._value


def cached_lambda(x: Callable[[], Any]) -> CachedLambda:
    return CachedLambda(x)
