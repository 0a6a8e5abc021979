"""Periodic evaluation (optimus_dl/recipe/train/mixins/managers/evaluation_manager.py:49-548).

For every evaluation dataset (sorted by name, each with its own ``eval_freq`` / ``eval_iterations``):
iterate its resettable loader under ``torch.no_grad`` and the AMP / FP8 forward context, log into
the meter group ``eval/{name}``, agree across ranks on exhaustion with an ``all_reduce(MAX)`` of a
flag (skipped when ``eval_guaranteed_same_batches``), optionally save per-rank mid-evaluation state
every ``eval_checkpointing`` batches and resume from it, then aggregate meters over ranks.
Returns ``{f"{prefix}/{name}": metrics}``."""

from __future__ import annotations

import contextlib
import logging
import time
from dataclasses import dataclass
from typing import Any

import torch

from .....core.profile import measured_next
from .....core.registry import RegistryConfig, make_registry
from .....metrics import MetricEngine
from .....metrics.base import compute_meters, meters_group, step_meters
from .....metrics.common import log_averaged, log_event_end, log_event_start, log_summed

logger = logging.getLogger(__name__)


@dataclass
class EvaluatorConfig(RegistryConfig):
    amp: Any = None


class Evaluator:
    def __init__(self, cfg: Any = None, eval_freq: int = 0, eval_iterations: int | None = None,
                 eval_guaranteed_same_batches: bool = False, eval_checkpointing: int | None = None,
                 metrics_config: Any = None, eval_checkpoint_manager: Any = None, output_path: Any = None,
                 **kwargs: Any):
        self.cfg = cfg
        self.eval_freq, self.eval_iterations = eval_freq, eval_iterations
        self.same_batches, self.eval_checkpointing = eval_guaranteed_same_batches, eval_checkpointing
        self.metrics_config = metrics_config or {}
        self.output_path = output_path
        if eval_checkpoint_manager is None and output_path is not None:
            from .....checkpoint.eval_checkpoint_manager import EvaluationCheckpointManager
            eval_checkpoint_manager = EvaluationCheckpointManager(output_path)
        self.eval_ckpt = eval_checkpoint_manager

    @property
    def eval_checkpoint_manager(self) -> Any:
        """The manager of mid-evaluation state (attribute name of
        optimus_dl/recipe/train/mixins/managers/evaluation_manager.py:96-99); settable."""
        return self.eval_ckpt

    @eval_checkpoint_manager.setter
    def eval_checkpoint_manager(self, manager: Any) -> None:
        self.eval_ckpt = manager

    def should_evaluate(self, iteration: int, pipeline: Any = None) -> bool:
        freq = (pipeline.eval_freq if pipeline is not None and pipeline.eval_freq is not None else self.eval_freq)
        return bool(freq) and freq > 0 and iteration % freq == 0

    def any_due(self, iteration: int, eval_data: dict[str, Any]) -> bool:
        return any(self.should_evaluate(iteration, p) for p in eval_data.values())

    def should_run_evaluation(self, iteration: int, eval_data_dict: dict[str, Any]) -> bool:
        """Whether any dataset is due at ``iteration`` (reference name of :meth:`any_due`; ``None`` entries are skipped)."""
        return self.any_due(iteration, {k: v for k, v in eval_data_dict.items() if v is not None})

    def run_evaluation_if_needed(self, iteration: int, model: torch.nn.Module, criterion: Any, eval_data_dict: dict[str, Any],
                                 device: Any = None, collective: Any = None, all_metrics_configs: Any = None,
                                 training_context: dict[str, Any] | None = None) -> dict | None:
        """Evaluate the datasets that are due at ``iteration``; ``None`` when none is
        (argument order of optimus_dl/recipe/train/mixins/managers/evaluation_manager.py:172-181)."""
        data = {k: v for k, v in eval_data_dict.items() if v is not None}
        if not self.any_due(iteration, data):
            return None
        if all_metrics_configs is not None:
            self.metrics_config = all_metrics_configs
        return self.run_evaluation(model, criterion, data, iteration, collective=collective, training_context=training_context)

    def cleanup_all_eval_checkpoints(self, iteration: int | None = None, exclude_iteration: int | None = None) -> None:
        if self.eval_ckpt is not None:
            self.eval_ckpt.cleanup(iteration=iteration, exclude_iteration=exclude_iteration)

    def forward_context(self, training_context: dict[str, Any] | None):
        if training_context is None:
            return contextlib.nullcontext()
        return training_context["amp_ctx"]()

    @torch.no_grad()
    def run_evaluation(self, model: torch.nn.Module, criterion: Any, eval_data_dict: dict[str, Any] | None = None,
                       device: Any = None, max_iterations: int | None = None, collective: Any = None,
                       all_metrics_configs: Any = None, metrics_prefix: str = "eval", show_progress: bool = False,
                       iteration: int | None = None, *, training_context: dict[str, Any] | None = None,
                       force: bool = False, prefix: str | None = None, eval_data: dict[str, Any] | None = None,
                       ) -> dict[str, dict[str, Any]]:
        """Evaluate the given datasets; ``{"<prefix>/<name>": metrics}``.

        Arguments up to ``iteration`` are those of optimus_dl/recipe/train/mixins/managers/evaluation_manager.py:
        246-258, in that order (``max_iterations`` caps datasets that set no ``eval_iterations`` of their own;
        ``all_metrics_configs`` replaces the evaluator's metric configs for this call). With ``iteration`` given and
        ``force`` false, datasets whose frequency does not divide it are skipped; without ``iteration`` everything
        given is evaluated, as there. The keyword-only arguments are this package's (``prefix`` / ``eval_data`` are
        earlier spellings of ``metrics_prefix`` / ``eval_data_dict``).
        """
        data = eval_data_dict if eval_data_dict is not None else (eval_data or {})
        if isinstance(device, int) and not isinstance(device, bool) and iteration is None:
            iteration, device = device, None      # earlier positional form: (model, criterion, data, iteration)
        if prefix is not None:
            metrics_prefix = prefix
        ckpt_iteration = iteration            # None: no mid-evaluation state is read or written
        if iteration is None:
            iteration, force = 0, True
        saved_cfg, saved_iters = self.metrics_config, self.eval_iterations
        if all_metrics_configs is not None:
            self.metrics_config = all_metrics_configs
        if max_iterations is not None:
            self.eval_iterations = max_iterations if max_iterations >= 0 else None
        was_training = model.training
        model.eval()
        results: dict[str, dict[str, Any]] = {}
        if device is None:
            device = training_context["device"] if training_context else next(model.parameters()).device
        try:
            for name in sorted(data):
                pipe = data[name]
                if pipe is None or (not force and not self.should_evaluate(iteration, pipe)):
                    continue
                results[f"{metrics_prefix}/{name}"] = self._evaluate_one(model, criterion, name, pipe, ckpt_iteration, collective,
                                                                         training_context, device, metrics_prefix)
        finally:
            model.train(was_training)
            self.metrics_config, self.eval_iterations = saved_cfg, saved_iters
        return results

    def _evaluate_one(self, model, criterion, name, pipe, ckpt_iteration, collective, ctx, device, prefix) -> dict[str, Any]:
        group = f"{prefix}/{name}"
        cfgs = self.metrics_config.get(name) if hasattr(self.metrics_config, "get") else None
        engine = MetricEngine(group, cfgs) if cfgs else None
        max_iters = pipe.eval_iterations if pipe.eval_iterations is not None else self.eval_iterations
        same = pipe.eval_guaranteed_same_batches if pipe.eval_guaranteed_same_batches is not None else self.same_batches
        ckpt_every = pipe.eval_checkpointing if pipe.eval_checkpointing is not None else self.eval_checkpointing
        world = collective.world_size if collective is not None else 1
        with meters_group(group, log_freq=1, force_recreate=True):
            t_start = time.perf_counter()
            log_event_start("perf/total_run")
            loader = getattr(pipe, "dataloader", pipe)
            restorable = loader if hasattr(loader, "load_state_dict") else None
            data_iter = iter(loader)
            processed = 0
            if self.eval_ckpt is not None and ckpt_iteration is not None:
                processed = self.eval_ckpt.load_iteration_state(
                    ckpt_iteration, name, group, eval_iter=restorable if restorable is not None else data_iter,
                    collective=collective)
                if processed:
                    if restorable is not None:
                        data_iter = iter(loader)
                    logger.info("resuming evaluation %s at batch %d", name, processed)
            requested = engine.required_external_protocols if engine is not None else None
            while max_iters is None or processed < max_iters:
                exhausted, batch = 0, None
                elapsed_batch_get = 0.0
                try:
                    elapsed_batch_get, batch = measured_next(data_iter)
                except StopIteration:
                    exhausted = 1
                if world > 1 and not same:
                    flag = torch.tensor([exhausted], dtype=torch.int32, device=device)
                    collective.all_reduce(flag, op=torch.distributed.ReduceOp.MAX)
                    exhausted = int(flag.item())
                if exhausted:
                    break
                log_event_start("perf/full_iteration")
                with self.forward_context(ctx):
                    loss, exposed = criterion(model, batch, requested_protocols=requested)
                if engine is not None:
                    engine.update(dict(model=model, batch=batch), exposed)
                log_event_end("perf/full_iteration")
                log_averaged("perf/batch_get", elapsed_batch_get)
                log_summed("num_batches", lambda: 1)
                step_meters(group)
                processed += 1
                if self.eval_ckpt is not None and ckpt_every and processed % int(ckpt_every) == 0:
                    assert ckpt_iteration is not None, "Iteration must be provided for checkpointing"
                    src = loader if hasattr(loader, "state_dict") else data_iter
                    self.eval_ckpt.save_iteration_state(ckpt_iteration, name, src.state_dict(), group, collective=collective,
                                                        eval_iterations_processed=processed)
            log_event_end("perf/total_run")
            total_ms = (time.perf_counter() - t_start) * 1e3
            log_averaged("perf/total_run_ms", total_ms, round=1)
            log_averaged("perf/ms_per_batch", total_ms / max(processed, 1), round=2)
        raw = compute_meters(group, aggregate=True, collective=collective)
        return engine.compute(raw) if engine is not None else raw


_R, register_evaluator, build_evaluator = make_registry("evaluator")
register_evaluator("base", EvaluatorConfig)(Evaluator)
