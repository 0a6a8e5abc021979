"""Timing helpers (optimus_dl/core/profile.py:37-226).

``measured_*`` return ``(elapsed_ms, value)``. Unlike the reference, device timing is a first-class
citizen here: ``DeviceTimer`` brackets a region with CUDA events on the current stream and
reports milliseconds without forcing a sync until the value is read.
DCGM sampling is optional and degrades to ``None`` when the bindings are absent.
"""

from __future__ import annotations

import logging
import time
from typing import Any, Callable, Iterable, Iterator

import torch

logger = logging.getLogger(__name__)


# ---------------------------------------------------------------------- NVTX ranges
_NVTX = None


def nvtx_enabled() -> bool:
    """NVTX ranges are emitted when ``OPTIMUS_NVTX=1`` and a CUDA device exists (off by default: zero cost)."""
    global _NVTX
    if _NVTX is None:
        import os

        _NVTX = os.environ.get("OPTIMUS_NVTX", "0") not in ("", "0", "false", "False") and torch.cuda.is_available()
    return _NVTX


class nvtx_range:
    """``with nvtx_range("train/forward"):`` marks a phase for timeline tools; a no-op unless enabled.
    Ranges are placed around the train step's phases and around every transformer block."""

    __slots__ = ("name", "on")

    def __init__(self, name: str):
        self.name, self.on = name, nvtx_enabled()

    def __enter__(self):
        if self.on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()
        return False


def measured_next(it: Iterator) -> tuple[float, Any]:
    t0 = time.perf_counter()
    v = next(it)
    return (time.perf_counter() - t0) * 1e3, v


def measured_iter(iterable: Iterable) -> Iterator[tuple[float, Any]]:
    it = iter(iterable)
    while True:
        try:
            yield measured_next(it)
        except StopIteration:
            return


def measured_lambda(f: Callable[[], Any], cuda_events: bool = False, enabled: bool = True) -> tuple[float | None, Any]:
    if not enabled:
        return None, f()
    if cuda_events and torch.cuda.is_available():
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        v = f()
        e.record()
        e.synchronize()
        return s.elapsed_time(e), v
    t0 = time.perf_counter()
    v = f()
    return (time.perf_counter() - t0) * 1e3, v


class DeviceTimer:
    """CUDA-event stopwatch; ``elapsed_ms()`` synchronises on the end event only."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._s = self._e = None
        self._t0 = 0.0
        self._host_ms = 0.0

    def __enter__(self) -> "DeviceTimer":
        if self.enabled:
            self._s, self._e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._s.record()
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc) -> None:
        if self.enabled:
            self._e.record()
        self._host_ms = (time.perf_counter() - self._t0) * 1e3

    def elapsed_ms(self) -> float:
        if self.enabled:
            self._e.synchronize()
            return self._s.elapsed_time(self._e)
        return self._host_ms


_dcgm_state: dict[str, Any] = {}


def setup_dcgm(gpu_id: int = 0) -> bool:
    """Start watching SM activity / occupancy at 1 Hz through an embedded DCGM engine, if available."""
    try:
        import pydcgm  # type: ignore
        import dcgm_fields  # type: ignore
        import dcgm_structs  # type: ignore

        handle = pydcgm.DcgmHandle(opMode=dcgm_structs.DCGM_OPERATION_MODE_AUTO)
        group = pydcgm.DcgmGroup(handle, groupName=f"optimus_{gpu_id}", groupType=dcgm_structs.DCGM_GROUP_EMPTY)
        group.AddGpu(gpu_id)
        fields = [dcgm_fields.DCGM_FI_PROF_SM_ACTIVE, dcgm_fields.DCGM_FI_PROF_SM_OCCUPANCY]
        fg = pydcgm.DcgmFieldGroup(handle, f"optimus_fields_{gpu_id}", fields)
        group.samples.WatchFields(fg, 1_000_000, 3600.0, 0)
        _dcgm_state.update(handle=handle, group=group, fg=fg, gpu=gpu_id, fields=fields)
        return True
    except Exception as e:  # bindings or daemon missing
        logger.debug("DCGM unavailable: %s", e)
        return False


def get_sm_metrics() -> dict[str, float] | None:
    if not _dcgm_state:
        return None
    try:
        vals = _dcgm_state["group"].samples.GetLatest(_dcgm_state["fg"]).values
        per_gpu = vals[_dcgm_state["gpu"]]
        f_active, f_occ = _dcgm_state["fields"]
        return {"gpu_sm_active_pct": 100.0 * per_gpu[f_active][-1].value,
                "gpu_sm_occupancy_pct": 100.0 * per_gpu[f_occ][-1].value}
    except Exception:
        return None


def teardown_dcgm() -> None:
    try:
        if _dcgm_state:
            _dcgm_state["group"].Delete()
    except Exception:
        pass
    _dcgm_state.clear()
