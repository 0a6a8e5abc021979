"""Train recipe (optimus_dl/recipe/train/base.py:78-665).

Order of operations in ``run()``: seed and numerics setup; device + collective; per-rank file logging;
model (builder + transforms), optimizer, scheduler, criterion, training context; train / eval data;
resume from ``output_path`` (or load ``load_checkpoint`` with its strategy); loggers on the master rank;
``init`` meters; barrier; if the last checkpoint was written *before* an evaluation that never
finished ("dirty" checkpoint, ``eval_finished: False``), run that evaluation first; then the loop
``for iteration in range(start, iterations + 1)``: one optimizer step, logging on logging steps,
evaluation (full checkpoint before, metadata-only checkpoint after, when ``eval_resumable``) or a
periodic checkpoint. ``KeyboardInterrupt`` writes a final checkpoint and marks loggers INTERRUPTED.
"""

from __future__ import annotations

import logging
import os
from typing import Any

import torch

from ...checkpoint import EvaluationCheckpointManager, build_checkpoint_manager
from ...core import conf
from ...core.device import setup_device_and_collective
from ...core.log import setup_logging, trange
from ...core.seed import set_seed
from ...loggers.base import RunStatus
from ...metrics import MetricEngine
from ...metrics.base import compute_meters, meters_group, reset_meters, step_meters
from ...metrics.common import log_event_end, log_event_start
from ..mixins.model_builder import build_model_builder
from .builders.criterion_builder import build_criterion_builder
from .builders.data_builder import build_data_builder
from .builders.optimizer_builder import build_optimizer_builder
from .builders.scheduler_builder import build_scheduler_builder
from .mixins.execution.context_mixin import TrainingContextMixin
from .mixins.execution.interruption_mixin import TrainingInterruptionMixin
from .mixins.execution.iteration_mixin import TrainingIterationMixin
from .mixins.managers.evaluation_manager import build_evaluator
from .mixins.managers.logger_manager import build_logger_manager

logger = logging.getLogger(__name__)


class TrainRecipe(TrainingContextMixin, TrainingIterationMixin, TrainingInterruptionMixin):
    def __init__(self, cfg: Any, **kwargs: Any):
        self.cfg = cfg
        c = cfg.common
        self.optimization_config = cfg.optimization
        self.output_path = str(c.output_path)
        self.model_builder = build_model_builder(cfg.model_builder, model_transforms=cfg.model_transforms)
        self.optimizer_builder = build_optimizer_builder(cfg.optimizer_builder, optimization_config=cfg.optimization)
        self.criterion_builder = build_criterion_builder(cfg.criterion_builder, criterion_config=cfg.criterion)
        self.data_builder = build_data_builder(cfg.data_builder, data_config=cfg.data, data_seed=c.data_seed)
        self.scheduler_builder = build_scheduler_builder(cfg.scheduler_builder, lr_scheduler_config=cfg.lr_scheduler,
                                                         optimization_config=cfg.optimization)
        self.logger_manager = build_logger_manager(cfg.logger_manager, loggers_config=cfg.loggers)
        self.checkpoint_manager = build_checkpoint_manager(cfg.checkpoint_manager, output_path=self.output_path)
        self.evaluator = None  # built in run(): it needs the rank for mid-evaluation checkpoints

    # ------------------------------------------------------------------ setup helpers
    def setup_context(self) -> None:
        c = self.cfg.common
        set_seed(int(c.seed), deterministic=bool(c.deterministic))
        # TF32 off, as in the reference: fp32 paths are the numerical oracle
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        try:
            torch.set_float32_matmul_precision("highest")
        except Exception:
            pass

    def _full_config(self) -> Any:
        return conf.to_container(self.cfg, resolve=True)

    # ------------------------------------------------------------------ delegation surface
    # One-line forwards to the injected builders and managers, under the names the reference's recipe exposes
    # (optimus_dl/recipe/train/base.py:168-262), so subclasses and scripts written against it keep working.
    def build_model(self, *args: Any, **kwargs: Any):
        return self.model_builder.build_model(*args, **kwargs)

    def build_optimizer(self, *args: Any, **kwargs: Any):
        return self.optimizer_builder.build_optimizer(*args, **kwargs)

    def build_lr_scheduler(self, *args: Any, **kwargs: Any):
        return self.scheduler_builder.build_lr_scheduler(*args, **kwargs)

    def build_criterion(self, *args: Any, **kwargs: Any):
        return self.criterion_builder.build_criterion(*args, **kwargs)

    def build_train_data(self, *args: Any, **kwargs: Any):
        return self.data_builder.build_train_data(*args, **kwargs)

    def build_eval_data(self, *args: Any, **kwargs: Any):
        return self.data_builder.build_eval_data(*args, **kwargs)

    def build_loggers(self, *args: Any, **kwargs: Any):
        return self.logger_manager.build_loggers(*args, **kwargs)

    def setup_loggers(self, experiment_name: str, full_config: dict | None = None, **_: Any):
        return self.logger_manager.setup_loggers(experiment_name, full_config if full_config is not None else self._full_config())

    def log_metrics_to_loggers(self, *args: Any, **kwargs: Any):
        return self.logger_manager.log_metrics_to_loggers(*args, **kwargs)

    def close_loggers(self, run_status: RunStatus = RunStatus.SUCCESS, *args: Any, **kwargs: Any):
        self.logger_manager.finished(run_status)
        return self.logger_manager.close_loggers(*args, **kwargs)

    def save_checkpoint_if_needed(self, *args: Any, **kwargs: Any):
        return self.checkpoint_manager.save_checkpoint_if_needed(*args, **kwargs)

    def save_checkpoint(self, *args: Any, **kwargs: Any):
        return self.checkpoint_manager.save_checkpoint(*args, **kwargs)

    def load_checkpoint_if_exists(self, *args: Any, **kwargs: Any):
        return self.checkpoint_manager.load_checkpoint_if_exists(*args, **kwargs)

    def load_checkpoint(self, *args: Any, **kwargs: Any):
        return self.checkpoint_manager.load_checkpoint(*args, **kwargs)

    def run_evaluation_if_needed(self, *args: Any, **kwargs: Any):
        return self.evaluator.run_evaluation_if_needed(*args, **kwargs)

    def validate_config(self) -> None:
        """Refuse configurations that cannot train (same checks as the reference's recipe)."""
        cfg = self.cfg
        for key in ("model", "data", "criterion", "optimization"):
            assert cfg.get(key) is not None, f"{key.capitalize()} configuration is required"
        assert int(cfg.optimization.iterations) > 0, "iterations must be positive"
        assert int(cfg.optimization.acc_steps) > 0, "acc_steps must be positive"
        assert int(cfg.common.log_freq) > 0, "log_freq must be positive"

    def _save(self, iteration: int, *, model, optimizer, lr_scheduler, collective, train_loader, persistent=True,
              metadata_only=False, extra=None) -> None:
        # nothing is persisted from a step in which a kernel's bounded wait ran out (the sharding engine keeps the
        # last good state in that case); afterwards the ranks meet on the host, because writing a checkpoint takes
        # a different time on every rank and the device-side waits of the next step are bounded
        engine = getattr(getattr(model, "module", model), "_sharding_engine", None)
        if engine is not None:
            engine.verify()
        self._save_checkpoint(iteration, model=model, optimizer=optimizer, lr_scheduler=lr_scheduler, collective=collective,
                              train_loader=train_loader, persistent=persistent, metadata_only=metadata_only, extra=extra)
        if engine is not None:
            engine.host_sync()

    def _save_checkpoint(self, iteration: int, *, model, optimizer, lr_scheduler, collective, train_loader, persistent=True,
                         metadata_only=False, extra=None) -> None:
        self.checkpoint_manager.save_checkpoint(
            iteration=iteration, model=model, optimizer=optimizer, lr_scheduler=lr_scheduler, collective=collective,
            full_config=self._full_config(), persistent=persistent, metadata_only=metadata_only, extra_metadata=extra,
            data_loaders={"train": train_loader} if train_loader is not None else None,
            grad_scaler=self._ctx["scaler"], logger_manager=self.logger_manager)

    # ------------------------------------------------------------------ run
    def run(self) -> None:
        cfg, c = self.cfg, self.cfg.common
        self.validate_config()
        self.setup_context()
        is_restart = self.checkpoint_manager.is_restart()
        with meters_group("init", log_freq=1):
            log_event_start("perf/init")
            setup = setup_device_and_collective(use_gpu=bool(c.use_gpu), config=c.distributed)
            device, collective = setup.device, setup.collective
            setup_logging(log_path=os.path.join(self.output_path, "logging", f"rank_{collective.rank}"))
            logger.info("rank %d / %d on %s (restart=%s)", collective.rank, collective.world_size, device, is_restart)
            self.evaluator = build_evaluator(
                cfg.evaluator, eval_freq=int(c.eval_freq), eval_iterations=c.eval_iterations,
                eval_guaranteed_same_batches=bool(c.eval_guaranteed_same_batches), eval_checkpointing=c.eval_checkpointing,
                metrics_config=cfg.metrics,
                eval_checkpoint_manager=EvaluationCheckpointManager(self.output_path, collective.rank))
            model = self.model_builder.build_model(cfg.model, collective=collective, device=device, is_restart=is_restart,
                                                   checkpoint_manager=self.checkpoint_manager)
            if getattr(model, "_sharding_engine", None) is None:
                model = model.to(device)
            optimizer = self.optimizer_builder.build_optimizer(model.make_parameter_groups())
            lr_scheduler = self.scheduler_builder.build_lr_scheduler(optimizer)
            criterion = self.criterion_builder.build_criterion(collective=collective)
            self._ctx = self.setup_training_context(device, cfg.optimization.get("amp"))
            train_pipe = self.data_builder.build_train_data(collective=collective, device=device)
            eval_data = self.data_builder.build_eval_data(collective=collective, device=device)
            train_loader = train_pipe.dataloader if train_pipe is not None else None
            common = dict(model=model, optimizer=optimizer, lr_scheduler=lr_scheduler, collective=collective,
                          data_loaders={"train": train_loader} if train_loader is not None else None,
                          grad_scaler=self._ctx["scaler"], logger_manager=self.logger_manager)
            start_iteration, metadata = self.checkpoint_manager.load_checkpoint_if_exists(**common)
            if metadata is None and c.load_checkpoint:
                strategy = c.load_checkpoint_strategy
                meta = self.checkpoint_manager.load_checkpoint(str(c.load_checkpoint), strategy=strategy, **common)
                if strategy.get("load_iteration", True):
                    start_iteration = int(meta["iteration"]) + 1
            if collective.is_master:
                self.logger_manager.build_loggers()
                self.logger_manager.setup_loggers(str(c.exp_name), self._full_config())
            log_event_end("perf/init")
        init_metrics = compute_meters("init", aggregate=True, collective=collective)
        if collective.is_master and init_metrics:
            self.logger_manager.log_metrics_to_loggers(init_metrics, start_iteration, "init")
        train_iter = iter(train_loader) if train_loader is not None else None
        engine_cfg = cfg.metrics.get("train") if cfg.metrics else None
        metric_engine = MetricEngine("train", engine_cfg) if engine_cfg else None
        collective.barrier()
        iterations = int(cfg.optimization.iterations)
        save_kw = dict(model=model, optimizer=optimizer, lr_scheduler=lr_scheduler, collective=collective,
                       train_loader=train_loader)
        status = RunStatus.FINISHED
        iteration = start_iteration - 1
        try:
            # a checkpoint written right before an evaluation that did not finish: redo the evaluation
            if metadata is not None and metadata.get("eval_finished") is False and eval_data:
                it0 = int(metadata["iteration"])
                logger.info("resuming the unfinished evaluation of iteration %d", it0)
                self._evaluate_and_log(model, criterion, eval_data, it0, collective, force=False)
                self._save(it0, metadata_only=True, extra={"eval_finished": True}, **save_kw)
                collective.barrier()
            for iteration in trange(start_iteration, iterations + 1, desc="train", disable=not collective.is_master):
                should_log = self.run_training_iteration(
                    model, optimizer, criterion, train_iter, self._ctx, lr_scheduler=lr_scheduler,
                    acc_steps=int(cfg.optimization.acc_steps), clip_grad_norm=cfg.optimization.get("clip_grad_norm"),
                    log_freq=int(c.log_freq), metric_engine=metric_engine, collective=collective)
                if should_log:
                    metrics = compute_meters("train", aggregate=True, collective=collective)
                    if metric_engine is not None:
                        metrics = metric_engine.compute(metrics)
                    if collective.is_master:
                        self.logger_manager.log_metrics_to_loggers(metrics, iteration, "train")
                        logger.info("iteration %d: %s", iteration,
                                    {k: v for k, v in metrics.items() if k in ("loss", "perplexity", "accuracy", "learning_rate")})
                step_meters("train")
                if should_log:
                    reset_meters("train")
                if eval_data and self.evaluator.any_due(iteration, eval_data):
                    if c.eval_resumable:
                        self._save(iteration, extra={"eval_finished": False}, **save_kw)
                    self._evaluate_and_log(model, criterion, eval_data, iteration, collective)
                    if c.eval_resumable:
                        self._save(iteration, metadata_only=True, extra={"eval_finished": True}, **save_kw)
                    collective.barrier()
                else:
                    persistent = bool(c.save_freq) and iteration % int(c.save_freq) == 0
                    last = bool(c.last_save_freq) and iteration % int(c.last_save_freq) == 0
                    if persistent or last:
                        self._save(iteration, persistent=persistent, **save_kw)
        except KeyboardInterrupt:
            status = RunStatus.INTERRUPTED
            self.handle_training_interruption(iteration, lambda it: self._save(it, persistent=False, **save_kw))
        except Exception:
            status = RunStatus.FAILED
            raise
        finally:
            if collective.is_master:
                self.logger_manager.finished(status)
                self.logger_manager.close_loggers()
            self.model, self.optimizer = model, optimizer
            try:
                collective.close()
            except Exception as e:
                logger.debug("collective.close: %s", e)

    def evaluate_and_log(self, iteration, model, criterion, eval_datapipeline, collective, device=None) -> dict:
        """Reference argument order for :meth:`_evaluate_and_log` (always evaluates)."""
        return self._evaluate_and_log(model, criterion, eval_datapipeline, iteration, collective, force=True)

    def _evaluate_and_log(self, model, criterion, eval_data, iteration, collective, force: bool = False) -> dict:
        results = self.evaluator.run_evaluation(model, criterion, eval_data, iteration, collective=collective,
                                                training_context=self._ctx, force=force)
        if collective.is_master:
            for group, metrics in results.items():
                self.logger_manager.log_metrics_to_loggers(metrics, iteration, group)
                logger.info("evaluation %s @ %d: %s", group, iteration,
                            {k: v for k, v in metrics.items() if k in ("loss", "perplexity", "accuracy")})
        if self.evaluator.eval_ckpt is not None:
            self.evaluator.eval_ckpt.cleanup()
        engine = getattr(getattr(model, "module", model), "_sharding_engine", None)
        if engine is not None:
            engine.host_sync()      # evaluation length differs per rank: meet on the host before the next train step
        return results
