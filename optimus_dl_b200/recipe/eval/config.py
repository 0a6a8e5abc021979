"""Evaluation recipe configuration (optimus_dl/recipe/eval/config.py:13-75)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

MISSING = "???"


@dataclass
class EvalCommonConfig:
    checkpoint_path: str | None = MISSING   # checkpoint directory or metadata file ...
    model: Any = None                       # ... or a model config to build (exactly one of the two)
    use_gpu: bool = True
    seed: int = 42
    tokenizer: Any = MISSING


@dataclass
class LMEvalConfig:
    tasks: list[str] = field(default_factory=lambda: ["hellaswag"])
    num_fewshot: int = 0
    batch_size: int = 1
    limit: int | None = None
    output_path: str | None = None
    reference_scoring: bool = False     # score as the reference's adapter does (see eval/model.py); not a reference field


@dataclass
class EvalConfig:
    common: EvalCommonConfig = field(default_factory=EvalCommonConfig)
    lm_eval: LMEvalConfig = field(default_factory=LMEvalConfig)


def validate(cfg: Any) -> None:
    """Same checks as the reference's ``EvalConfig.__post_init__``."""
    import os

    path = cfg.common.get("checkpoint_path") if hasattr(cfg.common, "get") else cfg.common.checkpoint_path
    if path == MISSING:
        raise ValueError("checkpoint_path is required")
    if path is not None and not (os.path.exists(str(path)) or os.path.exists(os.path.dirname(str(path)) or ".")):
        raise ValueError(f"Checkpoint path does not exist: {path}")
