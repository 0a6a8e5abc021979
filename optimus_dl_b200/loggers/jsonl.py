"""``jsonl``: one JSON line per logging event (optimus_dl/modules/loggers/jsonl.py:30-373).

Layout, as the reference writes it: ``{output_dir}/{filename}`` for the ``train`` group and
``{stem}_{group}.jsonl`` for every other group; when a file passes ``max_file_size_mb`` it becomes ``{stem}.1.jsonl``
(older parts move to ``.2``, ``.3``, ... and the oldest beyond ``max_rotated_files`` is deleted), so the newest lines are
always in the un-numbered file; the run config is dumped as ``{experiment}_config.json`` / ``.yaml`` at setup; the end
of the run appends a ``{"group": "final", "status": ...}`` line to ``{stem}_final.jsonl``. Each line carries ``step``,
``group``, an ISO ``timestamp`` (optional) and the metrics, dictionaries flattened one level as ``key_sub``.
"""

from __future__ import annotations

import json
import logging
import os
from dataclasses import dataclass
from datetime import datetime, timezone
from pathlib import Path
from typing import Any

import yaml

from . import register_metrics_logger
from .base import BaseMetricsLogger, RunStatus
from .config import MetricsLoggerConfig

logger = logging.getLogger(__name__)


@dataclass
class JsonlLoggerConfig(MetricsLoggerConfig):
    output_dir: str = "logs"
    filename: str = "metrics.jsonl"
    append_mode: bool = True                 # append to an existing file instead of truncating it
    flush_every: int = 10                    # flush + fsync every N lines
    include_timestamp: bool = True
    include_group_in_filename: bool = True   # one file per group other than "train"
    max_file_size_mb: float | None = 200     # rotate beyond this size; None / 0 = never
    max_rotated_files: int = -1              # numbered parts kept; <= 0 keeps all
    indent: int | None = None
    sort_keys: bool = False
    dump_config: bool = True                 # write the run config next to the metrics at setup


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
        self.output_dir = Path(os.path.expanduser(str(cfg.output_dir)))
        name = str(cfg.filename)
        self.stem, self.ext = (name.rsplit(".", 1) + ["jsonl"])[:2] if "." in name else (name, "jsonl")
        self._files: dict[str, Any] = {}
        self._paths: dict[str, Path] = {}
        self._writes = 0
        limit = cfg.get("max_file_size_mb")
        self._limit_bytes = float(limit) * 2**20 if limit else 0.0

    # ------------------------------------------------------------------ files
    def _path(self, group: str) -> Path:
        separate = bool(self.cfg.get("include_group_in_filename", True)) and bool(self.cfg.get("separate_groups", True))
        if separate and group not in ("train", "", None):
            safe = str(group).replace("/", "_").replace("\\", "_")
            return self.output_dir / f"{self.stem}_{safe}.{self.ext}"
        return self.output_dir / f"{self.stem}.{self.ext}"

    def _file(self, group: str):
        f = self._files.get(group)
        if f is None:
            self.output_dir.mkdir(parents=True, exist_ok=True)
            path = self._paths[group] = self._path(group)
            for other, p in self._paths.items():        # groups that share one file share one handle
                if other != group and p == path and other in self._files:
                    f = self._files[group] = self._files[other]
                    return f
            f = self._files[group] = open(path, "a" if self.cfg.get("append_mode", True) else "w", encoding="utf-8")
        return f

    def _rotate(self, group: str) -> None:
        """Current file -> ``.1``; ``.k`` -> ``.k+1``; parts beyond ``max_rotated_files`` are dropped."""
        f = self._files.get(group)
        if f is None:
            return
        f.flush()
        f.close()
        path = self._paths[group]
        sharing = [g for g, p in self._paths.items() if p == path and g in self._files]
        for g in sharing:
            self._files.pop(g)
        stem, ext, parent = path.stem, path.suffix, path.parent
        numbered = lambda i: parent / f"{stem}.{i}{ext}"  # noqa: E731
        keep = int(self.cfg.get("max_rotated_files", -1) or 0)
        if keep > 0:
            numbered(keep).unlink(missing_ok=True)
            top = keep - 1
        else:
            top = 0
            for p in parent.glob(f"{stem}.*{ext}"):
                tail = p.stem.rsplit(".", 1)[-1]
                if tail.isdigit():
                    top = max(top, int(tail))
        for i in range(top, 0, -1):
            if numbered(i).exists():
                numbered(i).rename(numbered(i + 1))
        path.rename(numbered(1))
        fresh = open(path, "a", encoding="utf-8")
        for g in sharing:
            self._files[g] = fresh

    # ------------------------------------------------------------------ logger interface
    def setup(self, experiment_name: str, config: dict[str, Any], logs_parent_path: str | None = None,
              start_iteration: int | None = None) -> None:
        if not self.enabled:
            return
        self.output_dir.mkdir(parents=True, exist_ok=True)
        self.experiment_name = experiment_name
        if self.cfg.get("dump_config", True):
            plain = _jsonable(config)
            try:
                with open(self.output_dir / f"{experiment_name}_config.json", "w") as f:
                    json.dump(plain, f, indent=2)
                with open(self.output_dir / f"{experiment_name}_config.yaml", "w") as f:
                    yaml.safe_dump(plain, f, sort_keys=False)
            except Exception as e:  # the run goes on without the config copy
                logger.error("could not write the config next to the metrics: %s", e)

    def _line(self, entry: dict[str, Any]) -> str:
        return json.dumps(entry, indent=self.cfg.get("indent"), sort_keys=bool(self.cfg.get("sort_keys", False)), default=str)

    def log_metrics(self, metrics: dict[str, Any], step: int, group: str = "train") -> None:
        if not self.enabled:
            return
        if self._limit_bytes and group in self._files and self._files[group].tell() > self._limit_bytes:
            self._rotate(group)
        entry: dict[str, Any] = {"step": step, "group": group}
        if self.cfg.get("include_timestamp", True):
            entry["timestamp"] = datetime.now(timezone.utc).isoformat()
        for key, value in metrics.items():
            if isinstance(value, dict):
                for sub, v in value.items():
                    entry[f"{key}_{sub}"] = _jsonable(v)
            else:
                entry[str(key)] = _jsonable(value)
        f = self._file(group)
        f.write(self._line(entry) + "\n")
        self._writes += 1
        every = int(self.cfg.get("flush_every", self.cfg.get("fsync_every", 10)) or 0)
        if every and self._writes % every == 0:
            f.flush()
            os.fsync(f.fileno())

    def finished(self, status: RunStatus = RunStatus.SUCCESS) -> None:
        if not self.enabled:
            return
        self.output_dir.mkdir(parents=True, exist_ok=True)
        entry: dict[str, Any] = {"step": None, "group": "final", "status": str(getattr(status, "value", status))}
        if self.cfg.get("include_timestamp", True):
            entry["timestamp"] = datetime.now(timezone.utc).isoformat()
        with open(self.output_dir / f"{self.stem}_final.jsonl", "a", encoding="utf-8") as f:
            f.write(self._line(entry) + "\n")

    def close(self) -> None:
        for f in {id(f): f for f in self._files.values()}.values():
            try:
                f.flush()
                f.close()
            except Exception:
                pass
        self._files.clear()

    def state_dict(self) -> dict[str, Any]:
        return {}       # files are found again by name; nothing else has to survive a restart

    def load_state_dict(self, state: dict[str, Any]) -> None:
        pass
