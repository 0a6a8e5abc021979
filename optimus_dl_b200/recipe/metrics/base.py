"""Metrics recipe: evaluate a model on datasets with the MetricEngine, outside of training
(optimus_dl/recipe/metrics/base.py:38-175). Order: seed, device + collective, model (checkpoint or
config + transforms), criterion, evaluation pipelines, loggers on the master rank, one evaluation
pass per dataset, results logged under ``eval/<dataset>`` at step 0 and returned."""

from __future__ import annotations

import logging
from typing import Any

from ...checkpoint import build_checkpoint_manager
from ...core import conf
from ...core.device import setup_device_and_collective
from ...core.seed import set_seed
from ..mixins.model_builder import build_model_builder
from ..train.builders.criterion_builder import build_criterion_builder
from ..train.builders.data_builder import build_data_builder
from ..train.mixins.managers.evaluation_manager import build_evaluator
from ..train.mixins.managers.logger_manager import build_logger_manager

logger = logging.getLogger(__name__)


class MetricsRecipe:
    def __init__(self, cfg: Any, **kwargs: Any):
        self.cfg = cfg
        c = cfg.common
        self.model_builder = build_model_builder(cfg.model_builder, model_transforms=cfg.model_transforms)
        self.data_builder = build_data_builder(cfg.data_builder, data_config=cfg.data, data_seed=c.data_seed,
                                               tokenizer_config=c.get("tokenizer"))
        self.criterion_builder = build_criterion_builder(cfg.criterion_builder, criterion_config=cfg.criterion)
        self.checkpoint_manager = build_checkpoint_manager(cfg.checkpoint_manager, output_path=str(c.output_path))
        self.logger_manager = build_logger_manager(cfg.logger_manager, loggers_config=cfg.loggers)
        self.evaluator = build_evaluator(cfg.evaluator, eval_freq=1, eval_iterations=c.get("max_iterations"),
                                         metrics_config=cfg.metrics)

    def run(self) -> dict[str, dict[str, Any]]:
        c = self.cfg.common
        set_seed(int(c.seed))
        setup = setup_device_and_collective(use_gpu=bool(c.use_gpu), config=c.distributed)
        device, collective = setup.device, setup.collective
        logger.info("metrics evaluation on %s", device)
        if c.get("checkpoint_path"):
            logger.info("loading model from checkpoint %s", c.checkpoint_path)
            model, _ = self.checkpoint_manager.build_model_from_checkpoint(str(c.checkpoint_path), device=device)
        else:
            assert self.cfg.model is not None, "Model config required if no checkpoint path provided"
            model = self.model_builder.build_model(self.cfg.model, collective=collective, device=device)
        model = model.to(device).eval()
        if collective.is_master:
            logger.info("model built: %s (parameters=%d)", type(model).__name__, sum(p.numel() for p in model.parameters()))
        criterion = self.criterion_builder.build_criterion(collective=collective)
        eval_data = self.data_builder.build_eval_data(device=device, collective=collective)
        if collective.is_master:
            self.logger_manager.build_loggers()
            self.logger_manager.setup_loggers(str(c.name), conf.to_container(self.cfg, resolve=True))
        results: dict[str, dict[str, Any]] = {}
        try:
            results = self.evaluator.run_evaluation(model, criterion, eval_data, iteration=0, collective=collective,
                                                    prefix="metrics", force=True)
            if collective.is_master:
                for name, metrics in results.items():
                    self.logger_manager.log_metrics_to_loggers(metrics, 0, f"eval/{name}")
        finally:
            if collective.is_master:
                self.logger_manager.close_loggers()
        return results
