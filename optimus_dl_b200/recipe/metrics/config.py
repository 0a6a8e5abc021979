"""Configuration of the metrics recipe (optimus_dl/recipe/metrics/config.py:32-112)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ...core.registry import RegistryConfigStrict
from ...parallel.collective import DistributedConfig

MISSING = "???"


@dataclass
class MetricsRecipeConfig:
    name: str = "metrics-eval"            # experiment name for the loggers
    seed: int = 42
    data_seed: int = 42
    output_path: str = "outputs/metrics"
    checkpoint_path: str | None = None    # model source; otherwise ``model`` is built from its config
    use_gpu: bool = True
    distributed: DistributedConfig = field(default_factory=DistributedConfig)
    max_iterations: int | None = None     # batches per dataset (None: until exhausted)
    tokenizer: Any = None


@dataclass
class MetricsConfig(RegistryConfigStrict):
    args: dict = field(default_factory=dict)
    common: MetricsRecipeConfig = field(default_factory=MetricsRecipeConfig)
    model: Any = None
    data: Any = MISSING
    criterion: Any = MISSING
    metrics: dict = field(default_factory=dict)       # dataset name -> metric configs
    model_transforms: list = field(default_factory=list)
    loggers: Any = None
    model_builder: Any = field(default_factory=lambda: {"_name": "base"})
    criterion_builder: Any = field(default_factory=lambda: {"_name": "base"})
    data_builder: Any = field(default_factory=lambda: {"_name": "base"})
    checkpoint_manager: Any = field(default_factory=lambda: {"_name": "base"})
    logger_manager: Any = field(default_factory=lambda: {"_name": "base"})
    evaluator: Any = field(default_factory=lambda: {"_name": "base"})
