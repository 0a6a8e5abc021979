"""``jsonl``: one JSON line per logging event into ``{output_dir}/metrics[_group].jsonl``
(optimus_dl/modules/loggers/jsonl.py:30-373): per-group files, size-based rotation, fsync every
N lines, the run config dumped as json + yaml at setup, a ``_final.jsonl`` record at the end."""

from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass
from typing import Any

import yaml

from . import register_metrics_logger
from .base import BaseMetricsLogger, RunStatus
from .config import MetricsLoggerConfig


@dataclass
class JsonlLoggerConfig(MetricsLoggerConfig):
    output_dir: str = "logs"
    filename: str = "metrics"
    max_file_size_mb: float | None = None
    fsync_every: int = 1
    separate_groups: bool = True
    dump_config: bool = True


def _jsonable(v: Any) -> Any:
    if isinstance(v, (str, int, float, bool)) or v is None:
        return v
    if isinstance(v, dict):
        return {str(k): _jsonable(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_jsonable(x) for x in v]
    if hasattr(v, "item"):
        try:
            return v.item()
        except Exception:
            pass
    return str(v)


@register_metrics_logger("jsonl", JsonlLoggerConfig)
class JsonlLogger(BaseMetricsLogger):
    def __init__(self, cfg, state_dict: dict | None = None, **kwargs: Any):
        super().__init__(cfg)
        self.output_dir = os.path.expanduser(str(cfg.output_dir))
        self._files: dict[str, Any] = {}
        self._lines: dict[str, int] = {}
        self._rotation: dict[str, int] = dict((state_dict or {}).get("rotation", {}))

    def _path(self, group: str) -> str:
        name = self.cfg.filename
        if self.cfg.separate_groups and group not in ("train", "", None):
            name = f"{name}_{str(group).replace('/', '_')}"
        rot = self._rotation.get(group, 0)
        if rot:
            name = f"{name}.{rot}"
        return os.path.join(self.output_dir, name + ".jsonl")

    def _file(self, group: str):
        f = self._files.get(group)
        if f is None:
            os.makedirs(self.output_dir, exist_ok=True)
            f = self._files[group] = open(self._path(group), "a", encoding="utf-8")
        return f

    def setup(self, experiment_name: str, config: dict[str, Any]) -> None:
        if not self.enabled:
            return
        os.makedirs(self.output_dir, exist_ok=True)
        if self.cfg.dump_config:
            with open(os.path.join(self.output_dir, "config.json"), "w") as f:
                json.dump(_jsonable(config), f, indent=2)
            with open(os.path.join(self.output_dir, "config.yaml"), "w") as f:
                yaml.safe_dump(_jsonable(config), f, sort_keys=False)
        self.experiment_name = experiment_name

    def log_metrics(self, metrics: dict[str, Any], step: int, group: str = "train") -> None:
        if not self.enabled:
            return
        rec = {"step": step, "group": group, "time": time.time(), **_jsonable(metrics)}
        f = self._file(group)
        f.write(json.dumps(rec) + "\n")
        n = self._lines[group] = self._lines.get(group, 0) + 1
        if self.cfg.fsync_every and n % int(self.cfg.fsync_every) == 0:
            f.flush()
            os.fsync(f.fileno())
        limit = self.cfg.max_file_size_mb
        if limit and f.tell() > float(limit) * 2**20:
            f.close()
            self._files.pop(group)
            self._rotation[group] = self._rotation.get(group, 0) + 1

    def finished(self, status: RunStatus = RunStatus.FINISHED) -> None:
        if not self.enabled:
            return
        os.makedirs(self.output_dir, exist_ok=True)
        with open(os.path.join(self.output_dir, f"{self.cfg.filename}_final.jsonl"), "a") as f:
            f.write(json.dumps({"status": str(getattr(status, "value", status)), "time": time.time()}) + "\n")

    def close(self) -> None:
        for f in self._files.values():
            try:
                f.flush()
                f.close()
            except Exception:
                pass
        self._files.clear()

    def state_dict(self) -> dict[str, Any]:
        return {"rotation": dict(self._rotation)}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self._rotation = dict(state.get("rotation", {}))
