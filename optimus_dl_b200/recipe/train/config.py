"""Train recipe configs (optimus_dl/recipe/train/config.py:41-242)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ...checkpoint.load_strategy import LoadStrategy
from ...core.registry import RegistryConfigStrict
from ...optim.config import OptimizationConfig
from ...parallel.collective import DistributedConfig


@dataclass
class TrainRecipeConfig:
    exp_name: str = "optimus-dl-run-${config_hash:}"
    exp_description: str | None = None
    exp_tags: list[str] = field(default_factory=list)
    log_freq: int = 16
    seed: int = 42
    data_seed: int = 42
    deterministic: bool = True
    eval_iterations: int | None = None
    eval_freq: int = 100
    eval_guaranteed_same_batches: bool = False
    eval_checkpointing: int | None = None
    eval_resumable: bool = True
    save_freq: int | None = "${.eval_freq}"  # type: ignore[assignment]
    last_save_freq: int | None = None
    output_path: str = "${oc.env:PERSISTENT_PATH,'./outputs'}/${.exp_name}"
    load_checkpoint: str | None = None
    load_checkpoint_strategy: LoadStrategy = field(default_factory=LoadStrategy)
    use_gpu: bool = True
    distributed: DistributedConfig = field(default_factory=DistributedConfig)


def _base(name: str = "base") -> dict:
    return {"_name": name}


@dataclass
class TrainConfig(RegistryConfigStrict):
    args: dict = field(default_factory=dict)
    common: TrainRecipeConfig = field(default_factory=TrainRecipeConfig)
    model: Any = "???"
    data: Any = "???"
    criterion: Any = "???"
    optimization: OptimizationConfig = "???"  # type: ignore[assignment]
    lr_scheduler: Any = None
    loggers: list[Any] | None = None
    metrics: dict[str, Any] = field(default_factory=dict)
    model_transforms: list[Any] = field(default_factory=list)
    model_builder: Any = field(default_factory=_base)
    optimizer_builder: Any = field(default_factory=_base)
    criterion_builder: Any = field(default_factory=_base)
    data_builder: Any = field(default_factory=_base)
    scheduler_builder: Any = field(default_factory=_base)
    logger_manager: Any = field(default_factory=_base)
    checkpoint_manager: Any = field(default_factory=_base)
    evaluator: Any = field(default_factory=_base)
