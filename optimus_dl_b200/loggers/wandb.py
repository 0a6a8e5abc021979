"""``wandb``: Weights & Biases logger; resumes a run by ``run_id``, uses ``iteration`` as the step metric,
uploads the logging directory as an artifact at the end (optimus_dl/modules/loggers/wandb.py:31-242).
Importing wandb is deferred, and a missing package disables the logger with a warning."""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Any

from . import register_metrics_logger
from .base import BaseMetricsLogger, RunStatus, flatten_metrics
from .config import MetricsLoggerConfig

logger = logging.getLogger(__name__)


@dataclass
class WandbLoggerConfig(MetricsLoggerConfig):
    project: str | None = None
    entity: str | None = None
    group: str | None = None
    name: str | None = None
    job_type: str | None = "train"
    mode: str | None = "online"        # "online" | "offline" | "disabled"
    save_code: bool = True
    log_dir_artifact: str | None = None
    dir: str | None = None


@register_metrics_logger("wandb", WandbLoggerConfig)
class WandbLogger(BaseMetricsLogger):
    def __init__(self, cfg, state_dict: dict | None = None, **kwargs: Any):
        super().__init__(cfg)
        self.run = None
        self.run_id = (state_dict or {}).get("run_id")
        self._wandb = None

    def setup(self, experiment_name: str, config: dict[str, Any], logs_parent_path: str | None = None,
              start_iteration: int | None = None) -> None:
        if not self.enabled:
            return
        try:
            import wandb
        except ImportError:
            logger.warning("wandb is not installed; the wandb logger is disabled")
            self.enabled = False
            return
        self._wandb = wandb
        kw: dict[str, Any] = dict(project=self.cfg.project, entity=self.cfg.entity, group=self.cfg.group,
                                  name=self.cfg.name or experiment_name, config=config, tags=list(self.cfg.tags or []),
                                  notes=self.cfg.notes, save_code=bool(self.cfg.save_code), dir=self.cfg.dir,
                                  job_type=self.cfg.get("job_type"))
        if self.cfg.mode:
            kw["mode"] = self.cfg.mode
        if self.run_id:
            kw.update(id=self.run_id, resume="allow")
        self.run = wandb.init(**{k: v for k, v in kw.items() if v is not None})
        self.run_id = self.run.id
        try:
            wandb.define_metric("iteration")
            wandb.define_metric("*", step_metric="iteration")
        except Exception:
            pass

    def log_metrics(self, metrics: dict[str, Any], step: int, group: str = "train") -> None:
        if not self.enabled or self.run is None:
            return
        flat = flatten_metrics(metrics, prefix=f"{group}/")
        flat["iteration"] = step
        self.run.log(flat)

    def finished(self, status: RunStatus = RunStatus.FINISHED) -> None:
        if self.run is None:
            return
        if self.cfg.log_dir_artifact and os.path.isdir(self.cfg.log_dir_artifact):
            try:
                art = self._wandb.Artifact(f"logs-{self.run.id}", type="logs")
                art.add_dir(self.cfg.log_dir_artifact)
                self.run.log_artifact(art)
            except Exception as e:
                logger.warning("could not upload log directory: %s", e)
        self._exit_code = 0 if status == RunStatus.FINISHED else 1

    def close(self) -> None:
        if self.run is not None:
            self.run.finish(exit_code=getattr(self, "_exit_code", 0))
            self.run = None

    def state_dict(self) -> dict[str, Any]:
        return {"run_id": self.run_id}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.run_id = state.get("run_id", self.run_id)
