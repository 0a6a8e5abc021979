"""Data pipeline configs (optimus_dl/modules/data/config.py:12-96)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..core.registry import RegistryConfig


@dataclass
class DataPipelineConfig:
    source: Any = None            # dataset registry config
    transform: Any = None         # transform registry config
    profile: bool = False
    report_freq: int = 100


@dataclass
class EvalDataPipelineConfig(DataPipelineConfig):
    eval_freq: int | None = None
    eval_iterations: int | None = None
    eval_guaranteed_same_batches: bool | None = None
    eval_checkpointing: int | None = None


@dataclass
class EvalDataConfig:
    eval_datasets: dict[str, Any] = field(default_factory=dict)
    scratch: Any = None


@dataclass
class DataConfig(EvalDataConfig):
    train_datasets: Any = None
