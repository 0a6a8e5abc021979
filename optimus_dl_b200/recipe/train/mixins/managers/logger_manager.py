"""Logger manager (optimus_dl/recipe/train/mixins/managers/logger_manager.py:30-206): builds every
configured logger on the master rank, fans metrics out, accounts the time spent logging, keeps
each logger's state under its ``id`` for checkpoints."""

from __future__ import annotations

import logging
import time
from dataclasses import dataclass
from typing import Any

from .....core.registry import RegistryConfig, make_registry
from .....loggers import build_metrics_logger
from .....loggers.base import RunStatus
from .....metrics.common import log_summed

logger = logging.getLogger(__name__)


@dataclass
class LoggerManagerConfig(RegistryConfig):
    pass


class LoggerManager:
    def __init__(self, cfg: Any = None, loggers_config: Any = None, **kwargs: Any):
        self.cfg = cfg
        self.loggers_config = list(loggers_config or [])
        self.loggers: list[Any] = []
        self._pending_state: dict[str, Any] = {}

    def build_loggers(self, **kwargs: Any) -> None:
        self.loggers = []
        for lc in self.loggers_config:
            if lc.get("enabled", True) is False:
                continue
            lid = str(lc.get("id") or lc.get("_name"))
            self.loggers.append(build_metrics_logger(lc, state_dict=self._pending_state.get(lid), **kwargs))

    def setup_loggers(self, experiment_name: str, config: dict[str, Any]) -> None:
        for lg in self.loggers:
            try:
                lg.setup(experiment_name, config)
            except Exception as e:
                logger.error("logger %s failed during setup: %s", type(lg).__name__, e)

    def log_metrics_to_loggers(self, metrics: dict[str, Any], step: int, group: str = "train") -> None:
        t0 = time.perf_counter()
        for lg in self.loggers:
            try:
                lg.log_metrics(metrics, step, group)
            except Exception as e:
                logger.error("logger %s failed: %s", type(lg).__name__, e)
        log_summed("ms_spent_logging", (time.perf_counter() - t0) * 1e3)

    def finished(self, status: RunStatus = RunStatus.FINISHED) -> None:
        for lg in self.loggers:
            try:
                lg.finished(status)
            except Exception as e:
                logger.error("logger %s failed in finished(): %s", type(lg).__name__, e)

    def close_loggers(self) -> None:
        for lg in self.loggers:
            try:
                lg.close()
            except Exception as e:
                logger.error("logger %s failed to close: %s", type(lg).__name__, e)

    def _id(self, lg: Any) -> str:
        return str(lg.cfg.get("id") or lg.cfg.get("_name"))

    def state_dict(self) -> dict[str, Any]:
        return {self._id(lg): lg.state_dict() for lg in self.loggers}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self._pending_state = dict(state or {})
        for lg in self.loggers:
            if self._id(lg) in self._pending_state:
                lg.load_state_dict(self._pending_state[self._id(lg)])


_R, register_logger_manager, build_logger_manager = make_registry("logger_manager")
register_logger_manager("base", LoggerManagerConfig)(LoggerManager)
