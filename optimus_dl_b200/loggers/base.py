"""Logger interface (optimus_dl/modules/loggers/base.py:18-111)."""

from __future__ import annotations

import enum
from typing import Any


class RunStatus(str, enum.Enum):
    """How a run ended (names and values of optimus_dl/modules/loggers/base.py:18-23; ``FINISHED`` / ``FAILED``
    are aliases of ``SUCCESS`` / ``FAILURE``)."""

    SUCCESS = "success"
    FAILURE = "failure"
    INTERRUPTED = "interrupted"
    FINISHED = "success"
    FAILED = "failure"


class BaseMetricsLogger:
    def __init__(self, cfg: Any, state_dict: dict | None = None, **kwargs: Any):
        self.cfg = cfg
        self.enabled = bool(cfg.get("enabled", True)) if cfg is not None else True

    def setup(self, experiment_name: str, config: dict[str, Any], logs_parent_path: str | None = None,
              start_iteration: int | None = None) -> None:
        """Called once on the master rank before training starts."""

    def log_metrics(self, metrics: dict[str, Any], step: int, group: str = "train") -> None:
        raise NotImplementedError

    def finished(self, status: RunStatus = RunStatus.FINISHED) -> None:
        """Mark the run's final status (before ``close``)."""

    def close(self) -> None:
        pass

    def state_dict(self) -> dict[str, Any]:
        return {}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        pass


def flatten_metrics(metrics: dict[str, Any], prefix: str = "") -> dict[str, Any]:
    out: dict[str, Any] = {}
    for k, v in metrics.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(flatten_metrics(v, key + "/"))
        else:
            out[key] = v
    return out
