"""``mlflow``: MLflow tracking logger (optimus_dl/modules/loggers/mlflow.py:37-395): resumes by
``run_id``, flattens and truncates params to MLflow's limits, logs the config as artifacts, tags the
run with environment details, optional async logging and system metrics. Importing mlflow is
deferred; a missing package disables the logger with a warning."""

from __future__ import annotations

import importlib.util
import json
import logging
import os
import platform
import subprocess
import tempfile
from dataclasses import dataclass
from typing import Any

from . import register_metrics_logger
from .base import BaseMetricsLogger, RunStatus, flatten_metrics
from .config import MetricsLoggerConfig

logger = logging.getLogger(__name__)
# whether the package can be imported at all (name of optimus_dl/modules/loggers/mlflow.py:28-34); the import
# itself still waits for ``setup``
MLFLOW_AVAILABLE = importlib.util.find_spec("mlflow") is not None
MAX_PARAM_LEN = 500
MAX_PARAMS_PER_CALL = 100


@dataclass
class MlflowLoggerConfig(MetricsLoggerConfig):
    tracking_uri: str | None = None
    experiment_name: str | None = None
    run_name: str | None = None
    # the reference's names (optimus_dl/modules/loggers/mlflow.py:55-66): ``project`` is the MLflow experiment,
    # ``name`` the run name; both win over the two fields above when set
    project: str | None = None
    name: str | None = None
    workspace: str | None = None
    artifact_location: str | None = None
    max_retries: int = 10
    backoff_factor: int = 2
    timeout: int = 15
    async_logging: bool = True
    log_system_metrics: bool = True
    log_config_artifacts: bool = True


def flatten_params(cfg: Any, prefix: str = "") -> dict[str, str]:
    out: dict[str, str] = {}
    if isinstance(cfg, dict):
        for k, v in cfg.items():
            out.update(flatten_params(v, f"{prefix}{k}."))
    elif isinstance(cfg, (list, tuple)):
        for i, v in enumerate(cfg):
            out.update(flatten_params(v, f"{prefix}{i}."))
    else:
        s = str(cfg)
        out[prefix[:-1]] = s if len(s) <= MAX_PARAM_LEN else s[: MAX_PARAM_LEN - 3] + "..."
    return out


def get_git_remote() -> str | None:
    """URL of ``origin`` of the working directory's repository, if any."""
    try:
        return subprocess.check_output(["git", "config", "--get", "remote.origin.url"], stderr=subprocess.DEVNULL,
                                       text=True).strip() or None
    except Exception:
        return None


def _git_commit() -> str | None:
    try:
        return subprocess.check_output(["git", "rev-parse", "HEAD"], stderr=subprocess.DEVNULL, text=True).strip()
    except Exception:
        return None


@register_metrics_logger("mlflow", MlflowLoggerConfig)
class MlflowLogger(BaseMetricsLogger):
    def __init__(self, cfg, state_dict: dict | None = None, **kwargs: Any):
        super().__init__(cfg)
        self.run_id = (state_dict or {}).get("run_id")
        self._mlflow = None
        self._active = False
        if self.enabled and not MLFLOW_AVAILABLE:
            logger.warning("mlflow is not installed; the mlflow logger is disabled")
            self.enabled = False

    def setup(self, experiment_name: str, config: dict[str, Any], logs_parent_path: str | None = None,
              start_iteration: int | None = None) -> None:
        if not self.enabled:
            return
        try:
            import mlflow
        except ImportError:
            logger.warning("mlflow is not installed; the mlflow logger is disabled")
            self.enabled = False
            return
        self._mlflow = mlflow
        if self.cfg.tracking_uri:
            mlflow.set_tracking_uri(self.cfg.tracking_uri)
        for var, value in (("MLFLOW_HTTP_REQUEST_MAX_RETRIES", self.cfg.max_retries),
                           ("MLFLOW_HTTP_REQUEST_BACKOFF_FACTOR", self.cfg.backoff_factor),
                           ("MLFLOW_HTTP_REQUEST_TIMEOUT", self.cfg.timeout)):
            try:
                getattr(mlflow.environment_variables, var).set(value)
            except Exception:
                os.environ[var] = str(value)
        workspace = self.cfg.workspace or os.getenv("MLFLOW_WORKSPACE")
        if workspace and hasattr(mlflow, "set_workspace"):
            try:
                mlflow.set_workspace(workspace)
            except Exception as e:
                logger.error("could not set the MLflow workspace: %s", e)
        exp_name = self.cfg.project or self.cfg.experiment_name or os.getenv("MLFLOW_EXPERIMENT_NAME") or experiment_name
        if self.cfg.artifact_location and mlflow.get_experiment_by_name(exp_name) is None:
            mlflow.create_experiment(exp_name, artifact_location=self.cfg.artifact_location)
        mlflow.set_experiment(exp_name)
        if self.cfg.async_logging:
            try:
                mlflow.config.enable_async_logging(True)
            except Exception:
                pass
        run = mlflow.start_run(run_id=self.run_id, run_name=self.cfg.name or self.cfg.run_name or experiment_name,
                               log_system_metrics=bool(self.cfg.log_system_metrics) or None)
        self.run_id = run.info.run_id
        self._active = True
        tags = {"host": platform.node(), "python": platform.python_version()}
        commit = _git_commit()
        if commit:
            tags["git_commit"] = commit
        for t in (self.cfg.tags or []):
            tags[str(t)] = "true"
        mlflow.set_tags(tags)
        params = list(flatten_params(config).items())
        for i in range(0, len(params), MAX_PARAMS_PER_CALL):
            try:
                mlflow.log_params(dict(params[i:i + MAX_PARAMS_PER_CALL]))
            except Exception as e:   # resumed runs may already hold these params
                logger.debug("log_params: %s", e)
        if self.cfg.log_config_artifacts:
            with tempfile.TemporaryDirectory() as d:
                p = os.path.join(d, "config.json")
                with open(p, "w") as f:
                    json.dump(config, f, indent=2, default=str)
                mlflow.log_artifact(p)

    def log_metrics(self, metrics: dict[str, Any], step: int, group: str = "train") -> None:
        if not self.enabled or not self._active:
            return
        flat = {k: float(v) for k, v in flatten_metrics(metrics, prefix=f"{group}/").items()
                if isinstance(v, (int, float)) and not isinstance(v, bool)}
        if flat:
            self._mlflow.log_metrics(flat, step=step)

    def finished(self, status: RunStatus = RunStatus.FINISHED) -> None:
        self._status = {"success": "FINISHED", "failure": "FAILED", "interrupted": "KILLED"}[str(getattr(status, "value", status))]

    def close(self) -> None:
        if self._active:
            self._mlflow.end_run(status=getattr(self, "_status", "FINISHED"))
            self._active = False

    def state_dict(self) -> dict[str, Any]:
        return {"run_id": self.run_id}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.run_id = state.get("run_id", self.run_id)


get_git_commit_hash = _git_commit   # the reference's name
