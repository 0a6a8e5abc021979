"""Device selection and collective bootstrap (optimus_dl/core/device.py:30-94)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch


@dataclass
class DeviceSetup:
    device: torch.device
    collective: Any


def get_best_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda")
    if getattr(torch.backends, "mps", None) is not None and torch.backends.mps.is_available():
        return torch.device("mps")
    if hasattr(torch, "xpu") and torch.xpu.is_available():
        return torch.device("xpu")
    return torch.device("cpu")


def setup_device_and_collective(use_gpu: bool = True, config: Any = None) -> DeviceSetup:
    from ..parallel.collective import build_best_collective

    device = get_best_device() if use_gpu else torch.device("cpu")
    collective = build_best_collective(config, device)
    if device.type == "cuda":
        device = torch.device("cuda", collective.local_rank)
        torch.cuda.set_device(device)
    return DeviceSetup(device=device, collective=collective)
