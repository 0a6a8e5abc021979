"""Process-global meter groups (optimus_dl/modules/metrics/base.py:30-759).

Code anywhere calls ``log_meter`` (or the helpers in ``metrics.common``) inside an active
``meters_group(name, log_freq)`` context. Values may be callables: they are evaluated only when
the group is going to log at this step, and the time spent evaluating them is billed to the
``ms_spent_logging`` meter. ``compute_meters(name, aggregate=True, collective=...)`` gathers every
rank's meter states with one object all-gather and merges them per meter.
"""

from __future__ import annotations

import time
from abc import ABC, abstractmethod
from collections import Counter, OrderedDict
from contextlib import contextmanager
from typing import Any, Callable, Generator


class BaseMeter(ABC):
    """A mergeable accumulator with a serialisable state."""

    @abstractmethod
    def compute(self) -> Any: ...

    @abstractmethod
    def log(self, **kwargs: Any) -> Any: ...

    @abstractmethod
    def merge(self, other_state: dict[str, Any]) -> None: ...

    def state_dict(self) -> dict[str, Any]:
        return {k: v for k, v in self.__dict__.items()}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.__dict__.update(state_dict)

    @classmethod
    def from_state_dict(cls, state_dict: dict[str, Any]) -> "BaseMeter":
        try:
            m = cls()
        except TypeError:                   # a meter whose constructor needs arguments: the state supplies everything
            m = cls.__new__(cls)
        m.load_state_dict(state_dict)
        return m


def _meter_class(name: str) -> type:
    """Meter class by the name a state was saved under: the bare class name of any ``BaseMeter`` subclass that has
    been imported, or a dotted path."""
    if "." in name:
        from ..core.conf import locate

        return locate(name)
    from . import common  # noqa: F401  (defines the stock meters)

    todo = list(BaseMeter.__subclasses__())
    while todo:
        cls = todo.pop()
        if cls.__name__ == name:
            return cls
        todo.extend(cls.__subclasses__())
    raise KeyError(f"unknown meter class {name!r}")


class MeterEntry:
    def __init__(self, meter: BaseMeter, reset: bool = False, priority: int = 0):
        self.meter, self.reset, self.priority = meter, reset, priority

    def state_dict(self) -> dict[str, Any]:
        return {"meter_class": type(self.meter).__name__, "meter": self.meter.state_dict(),
                "reset": self.reset, "priority": self.priority}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        self.meter = _meter_class(sd["meter_class"]).from_state_dict(sd["meter"])
        self.reset, self.priority = sd["reset"], sd["priority"]

    @classmethod
    def from_state_dict(cls, sd: dict[str, Any]) -> "MeterEntry":
        e = cls.__new__(cls)
        e.load_state_dict(sd)
        return e


class MeterGroup:
    def __init__(self, name: str, log_freq: int | None = None, log_logger_overhead: bool | None = None):
        self.name = name
        self.log_freq = 1 if log_freq is None else log_freq
        self.log_logger_overhead = True if log_logger_overhead is None else log_logger_overhead
        self._meters: "OrderedDict[str, MeterEntry]" = OrderedDict()
        self._iteration = 0

    @property
    def meters(self) -> "OrderedDict[str, MeterEntry]":
        return self._meters

    @property
    def _keys_sorted(self) -> list[str]:
        """Meter names in reporting order (priority, then name)."""
        return list(self._meters)

    @property
    def _iteration_counter(self) -> int:
        return self._iteration

    def should_log(self) -> bool:
        """Whether the current step is a logging step: the first one, and every ``log_freq``-th after it."""
        if not self.log_freq:
            return True
        return self._iteration % self.log_freq == 0

    def step(self) -> bool:
        """Advance the iteration counter; returns whether the step that now begins is a logging step."""
        self._iteration += 1
        return self.should_log()

    def add_meter(self, name: str, entry: MeterEntry) -> None:
        self._meters[name] = entry
        self._meters = OrderedDict(sorted(self._meters.items(), key=lambda kv: (kv[1].priority, kv[0])))

    def get_meter(self, name: str) -> MeterEntry | None:
        return self._meters.get(name)

    def compute(self) -> dict[str, Any]:
        return {k: e.meter.compute() for k, e in self._meters.items()}

    def reset(self) -> None:
        for k in [k for k, e in self._meters.items() if e.reset]:
            del self._meters[k]

    def state_dict(self) -> dict[str, Any]:
        return {"name": self.name, "log_freq": self.log_freq, "iteration_counter": self._iteration,
                "meters": {k: e.state_dict() for k, e in self._meters.items()}}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        self.log_freq = sd.get("log_freq", self.log_freq)
        self._iteration = sd.get("iteration_counter", sd.get("iteration", 0))
        self._meters = OrderedDict((k, MeterEntry.from_state_dict(v)) for k, v in sd.get("meters", {}).items())


_meter_groups: dict[str, MeterGroup] = {}
_active_meter_groups: Counter = Counter()


@contextmanager
def meters_group(name: str, log_freq: int | None = None, force_recreate: bool = False,
                 log_logger_overhead: bool | None = None) -> Generator[bool, None, None]:
    """Activate group ``name``; yields whether this step is a logging step."""
    if force_recreate:
        _meter_groups.pop(name, None)
    if name not in _meter_groups:
        _meter_groups[name] = MeterGroup(name, log_freq=log_freq, log_logger_overhead=log_logger_overhead)
    g = _meter_groups[name]
    if log_freq is not None:
        g.log_freq = log_freq
    if log_logger_overhead is not None:
        g.log_logger_overhead = log_logger_overhead
    _active_meter_groups[name] += 1
    try:
        yield g.should_log()
    finally:
        _active_meter_groups[name] -= 1
        if _active_meter_groups[name] <= 0:
            _active_meter_groups.pop(name, None)


def get_group(name: str) -> MeterGroup | None:
    return _meter_groups.get(name)


def compute_meters(name: str, aggregate: bool = False, collective: Any = None) -> dict[str, Any]:
    """Values of group ``name``; with ``aggregate`` (and a collective) every rank's meter states are merged first.
    Aggregated values come from freshly built meters and therefore carry no rounding, whatever ``round`` the logging
    call named: that is what optimus_dl/modules/metrics/base.py:531-556 reports (a one-rank collective included), and
    so what ends up in the logs of a training run."""
    g = _meter_groups.get(name)
    if g is None:
        local_states: dict[str, Any] = {}
    else:
        local_states = {k: e.state_dict() for k, e in g.meters.items()}
    if not aggregate or collective is None:
        return g.compute() if g is not None else {}
    all_states = [local_states] if collective.world_size == 1 else collective.all_gather_objects(local_states)
    merged: "OrderedDict[str, MeterEntry]" = OrderedDict()
    for rank_states in all_states:
        for k, sd in rank_states.items():
            if "meter_class" not in sd:
                # a bare meter state (what optimus_dl/modules/metrics/base.py:519-523 gathers): the class and
                # the priority are those of this rank's meter of the same name
                local = g.meters.get(k) if g is not None else None
                if local is None:
                    continue
                sd = {"meter": sd, "meter_class": type(local.meter).__name__, "reset": local.reset,
                      "priority": local.priority}
            if k not in merged:
                merged[k] = MeterEntry.from_state_dict(sd)
                if getattr(merged[k].meter, "round", None) is not None:
                    merged[k].meter.round = None
            else:
                merged[k].meter.merge(sd["meter"])
    ordered = sorted(merged.items(), key=lambda kv: (kv[1].priority, kv[0]))
    return {k: e.meter.compute() for k, e in ordered}


def step_meters(name: str) -> None:
    g = _meter_groups.get(name)
    if g is not None:
        g.step()


def reset_meters(name: str) -> None:
    g = _meter_groups.get(name)
    if g is not None:
        g.reset()


def state_dict() -> dict[str, Any]:
    return {k: g.state_dict() for k, g in _meter_groups.items()}


def load_state_dict(sd: dict[str, Any]) -> None:
    for k, gsd in sd.items():
        g = _meter_groups.setdefault(k, MeterGroup(k))
        g.load_state_dict(gsd)


def clear_all() -> None:
    """Drop every group (tests)."""
    _meter_groups.clear()
    _active_meter_groups.clear()


def _evaluate_value(v: Any) -> Any:
    if callable(v):
        v = v()
    try:
        import torch

        if isinstance(v, torch.Tensor) and v.numel() == 1:
            return v.item()
    except ImportError:
        pass
    return v


def log_meter(name: str, meter_factory: Callable[[], BaseMeter], reset: bool = True, priority: int = 100,
              force_log: bool = False, **kwargs: Any) -> None:
    """Feed ``kwargs`` to meter ``name`` of every active group that logs at this step."""
    force_log = force_log or not reset
    for gname in list(_active_meter_groups):
        g = _meter_groups[gname]
        if not (g.should_log() or force_log):
            continue
        if g.log_logger_overhead:
            t0 = time.perf_counter()
            vals = {k: _evaluate_value(v) for k, v in kwargs.items()}
            spent = (time.perf_counter() - t0) * 1e3
            if "ms_spent_logging" not in g.meters:
                from .common import SummedMeter

                g.add_meter("ms_spent_logging", MeterEntry(SummedMeter(), reset=True, priority=100))
            g.meters["ms_spent_logging"].meter.log(value=spent)
        else:
            vals = {k: _evaluate_value(v) for k, v in kwargs.items()}
        if name not in g.meters:
            g.add_meter(name, MeterEntry(meter_factory(), reset=reset, priority=priority))
        g.meters[name].meter.log(**vals)
