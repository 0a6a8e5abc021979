"""Metrics loggers and the ``metrics_logger`` registry (``_name``: jsonl, wandb, mlflow)."""

from ..core.bootstrap import bootstrap_module
from ..core.registry import make_registry
from .base import BaseMetricsLogger, RunStatus
from .config import MetricsLoggerConfig

_LOGGERS_REGISTRY, register_metrics_logger, build_metrics_logger = make_registry("metrics_logger", BaseMetricsLogger)
bootstrap_module(__name__)
