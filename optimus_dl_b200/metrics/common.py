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
        self.round, self.value = round, -float("inf")

    def log(self, value: float) -> None:
        self.value = max(self.value, value)

    def compute(self) -> float:
        """The largest value seen; before anything was logged the identity element itself (``-inf``), as
        optimus_dl/modules/metrics/common.py:121-130 returns it."""
        if not math.isfinite(self.value):
            return self.value
        return safe_round(self.value, self.round)

    def merge(self, other_state: dict[str, Any]) -> None:
        if other_state["value"] is not None:
            self.value = max(self.value, other_state["value"])


class MinMeter(MaxMeter):
    """The smallest value seen (``+inf`` before anything was logged). Kept as the maximum of the negated values, so
    ``value`` in the state is the NEGATED minimum, as in optimus_dl/modules/metrics/common.py:146-180: states and
    cross-rank merges are interchangeable with it."""

    def log(self, value: float) -> None:
        super().log(-value)

    def compute(self) -> float:
        return -super().compute()


class _IntervalMeter(BaseMeter):
    """Shared state of the two timing meters: ``elapsed`` nanoseconds over ``counter`` intervals; the result is the mean
    interval in milliseconds. The wall-clock anchor is not part of the state that survives a restart."""

    _ANCHOR = "start"

    def __init__(self, round: int | None = None):
        self.round, self.elapsed, self.counter = round, 0, 0
        setattr(self, self._ANCHOR, None)

    def compute(self) -> float:
        return safe_round(self.elapsed / self.counter / 1e6, self.round) if self.counter else 0

    def merge(self, other_state: dict[str, Any]) -> None:
        self.elapsed += other_state["elapsed"]
        self.counter += other_state["counter"]

    def state_dict(self) -> dict[str, Any]:
        return {"round": self.round, "elapsed": self.elapsed, "counter": self.counter}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.round = state_dict.get("round")
        if "total_ms" in state_dict:            # states written before the fields were renamed
            self.elapsed, self.counter = int(state_dict["total_ms"] * 1e6), int(state_dict.get("count", 0))
        else:
            self.elapsed, self.counter = state_dict.get("elapsed", 0), state_dict.get("counter", 0)
        setattr(self, self._ANCHOR, None)


class FrequencyMeter(_IntervalMeter):
    """Mean time between occurrences of an event, in milliseconds. The first occurrence only sets the anchor."""

    _ANCHOR = "start"

    def log(self) -> None:
        now = time.perf_counter_ns()
        if self.start is not None:
            self.elapsed += now - self.start
            self.counter += 1
        self.start = now


class StopwatchMeter(_IntervalMeter):
    """Mean duration between ``start`` and ``end`` events, in milliseconds."""

    _ANCHOR = "_start"

    def log(self, mode: str) -> None:
        assert mode in ("start", "end"), f"Unknown mode {mode!r}"
        if mode == "start":
            self.start()
        elif self._start is not None:           # an "end" event whose start was lost to a restart is dropped
            self.end()

    def start(self) -> None:
        self._start = time.perf_counter_ns()

    def end(self) -> None:
        assert self._start is not None, "Stopwatch was never started"
        self.elapsed += time.perf_counter_ns() - self._start
        self.counter += 1
        self._start = None


class AveragedExponentMeter(BaseMeter):
    """``exp(weighted mean(value))`` -- perplexity from mean loss. The mean lives in an inner :class:`AverageMeter`;
    the state is ``{"internal": <its state>, "round": ...}`` (optimus_dl/modules/metrics/common.py:398-452)."""

    def __init__(self, round: int | None = None):
        self._internal = AverageMeter()
        self.round = round

    @property
    def sum(self) -> float:
        return self._internal.sum

    @property
    def count(self) -> float:
        return self._internal.count

    def log(self, value: float, weight: float = 1.0) -> None:
        self._internal.log(value, weight)

    def compute(self) -> float:
        if not self._internal.count:
            return 0.0
        try:
            return safe_round(math.exp(self._internal.sum / self._internal.count), self.round)
        except OverflowError:
            return float("inf")

    @staticmethod
    def _inner(state: dict[str, Any]) -> dict[str, Any]:
        return state["internal"] if "internal" in state else {"sum": state["sum"], "count": state["count"], "round": None}

    def merge(self, other_state: dict[str, Any]) -> None:
        self._internal.merge(self._inner(other_state))

    def state_dict(self) -> dict[str, Any]:
        return {"internal": self._internal.state_dict(), "round": self.round}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self._internal.load_state_dict(self._inner(state_dict))
        self.round = state_dict.get("round")


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
